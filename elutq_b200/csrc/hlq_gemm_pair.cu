// Dequantize + tensor-core GEMM over HLQ weights for prefill on CTA PAIRS, sm_100a.
//
// Replaces the reference's prefill path, which runs one GEMV per token and re-streams all
// weights m times (C++/ops/src/arm/arm_gemm.cpp:362-387).  dequant_gemm_kernel (hlq_gemm.cu) moves
// both operands through shared memory: the dequantizers write the fp16 weight tile there and
// the tensor cores read it back, which together with the nibble-table lookups keeps the
// load/store pipe busier than the tensor pipe.  Here the weight operand never touches shared
// memory, and two CTAs on neighbouring SMs (a cluster of two) share the token tile:
//   * a pair owns tiles of 256 weight rows x up to 256 tokens and walks its share of them
//     (persistent: tile = pair, pair + pairs, ...; token tiles in groups that fit L2, inside a group
//     a row tile's token tiles one after the other); CTA c of the pair dequantizes rows 128 c .. 128 c + 127
//     straight from registers into its own TENSOR MEMORY (tcgen05.st, one lane = one row, a column
//     = two channels), four K steps of 128 channels deep = one slice of the streaming layout;
//   * each CTA brings in HALF of the token tile of a K step by TMA (two boxes of 64 channels,
//     128-byte swizzle); the copies of both CTAs complete on a barrier of CTA 0
//     (cp.async.bulk.tensor ... cta_group::2), the same barrier the dequantizer warps of both
//     CTAs arrive on: one wait per K step tells the issuing thread that both operands are there;
//   * threads of CTA 0 issue tcgen05.mma.cta_group::2 (256 x tokens x 16, A from tensor memory of
//     both SMs, B from shared memory of both SMs) and commit each stage free in both CTAs;
//   * both CTAs read their 128 x tokens accumulator back and store y[token][row] (+ bias); the
//     stages and barrier phases run on across tiles, so while one tile is read back the first
//     operands of the next are already in place and the tensor cores wait for the read-back only.
// Shared memory carries 32 KB per K step of 128 channels and SM, a quarter of the single-CTA kernel's.
//
//   warp 0        TMA producer (one thread)
//   warp 1        tensor memory allocation
//   warps 1, 2    in CTA 0 one thread of each issues the products, K steps in turn
//   warps 4..19   dequantizers, then epilogue: warp w owns lanes 32 (w & 3) .. +31 of tensor
//                 memory (= rows of the tile) and quarter (w - 4) >> 2 of every slice of 512
//                 channels = one of the four K steps in flight: a lane's unit of work is the
//                 streaming layout's unit, 16 bytes per plane = 128 channels of a row
//
// Measured on a B200 (w2g64, 2048 tokens): 13824x5120 1.41 PFLOP/s, 5120x5120 1.10, 5120x13824 1.21
// (dequant_gemm_kernel: 1.14, 0.72, 0.80); tensor pipe 75 % active.  What it was bound by on
// the way, each found with cycle counters in the issuing thread and one dequantizer warp:
// per-launch address arithmetic and 2-byte loads (a lane now loads 16 bytes per plane and slice),
// two barrier waits and 64-channel steps (now one wait per 128 channels), a single issuing
// thread whose waits and commits left the pipe idle (now two, alternating), tiles launched as
// CTAs (now persistent).
//
// Precision and operand formats as in hlq_gemm.cu.  All waits are bounded (poll limit); the first
// that runs out sets the CTA's failure flag, later waits give up at once, both CTAs still meet at
// the cluster barriers and tensor memory is always released.
#include <cuda.h>

#include "hlq_gemm_dev.cuh"

namespace hlq {
namespace gemm {

namespace {

constexpr uint32_t kByteTableBytes = 4096;                      // byte tables of two- and three-plane weights
constexpr int kPairStepK = 128;                                  // channels per K step: a quarter of a slice
constexpr int kPairStages = 4;                                   // K steps in flight (both operands): one slice
constexpr int kPairDeqWarps = 16;
constexpr int kPairThreads = 128 + 32 * kPairDeqWarps;
constexpr uint32_t kPairXBox = (kMaxTileM / 2) * kTileK * 2;     // 16 KB: half a token tile x 64 channels (one TMA box)
constexpr uint32_t kPairXStage = 2 * kPairXBox;                  // two boxes: 128 channels
constexpr uint32_t kPairDynSmem = 1024 + kPairStages * kPairXStage + kLutBytes + kBarBytes;
constexpr uint32_t kPairAccCols = 256, kPairACols = kPairStepK / 2;   // accumulator; one K step of the weight operand
constexpr uint32_t kPairTmemCols = 512;
static_assert(256 + kByteTableBytes <= kLutBytes, "tables");
static_assert(kPairStages * kPairStepK == 512, "the ring of K steps is one slice of the streaming layout");
static_assert(kPairAccCols + kPairStages * kPairACols <= kPairTmemCols, "tensor memory of one SM");
static_assert(8 * (2 * kPairStages + 4) + 16 <= kBarBytes, "barriers");

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// false when the wait gave up; once the CTA's flag is set every wait tries once
__device__ __forceinline__ bool pair_wait(uint32_t mbar, uint32_t parity, volatile int *fail) {
    if (mbar_try_wait(mbar, parity)) return true;
    if (!*fail)
        for (int i = 0; i < kSpinLimit; ++i) {
            if (mbar_try_wait(mbar, parity)) return true;
            if ((i & 255) == 255 && *fail) break;
        }
    *fail = 1;
    return false;
}
// this CTA's half of the token tile; completion is counted on `cluster_mbar` (a barrier of CTA 0)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, int c0, int c1,
                                                 uint32_t cluster_mbar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(cluster_mbar) : "memory");
}
// kind::f16, fp32 accumulator, A and B fp16, both K-major, M = 256 over the pair, N = tokens per tile
__device__ __forceinline__ uint32_t pair_idesc(int tile_m) {
    return (1u << 4) | ((uint32_t)(tile_m >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}
__device__ __forceinline__ void umma_f16_ts_pair(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                                 uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the barrier at `cluster_mbar` (of either CTA) once the products issued so far are done
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_mbar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_mbar)
                 : "memory");
}

// ---- two- and three-plane weights: a byte of a plane (8 channels) is looked up whole --------------
// Two planes: entry b of table p is, for the 8 channels of plane byte b, one selector byte per
// channel (.x channels 0..3, .y channels 4..7): 0x10 + 0x22 bit for plane 0, 0x44 bit for plane 1;
// the OR of the two entries selects, per pair of channels, the fp16 values z + b0 a0 + b1 a1 out of
// the 8 bytes {v0, v1, v2, v3} with one prmt.
// Three planes: entry b of table p is the byte's 8 bits spread to bit p of 8 nibbles; the OR of the
// three entries is the 3-bit code of 8 channels, which indexes byte tables of the 8 possible values
// (their low bytes in two registers, their high bytes in two): two prmt gather 4 low and 4 high
// bytes, two more pair them up.
// Either way a weight costs about half the ALU instructions of the nibble-mask form and the 2^q
// values of a group are rounded to fp16 once, from fp32.
template <int Q>
__device__ __forceinline__ void fill_byte_tables(int tid, int nthreads, unsigned char *tab) {
    if constexpr (Q == 2) {
        uint2 *t = (uint2 *)tab;                       // [plane][256]
        for (int e = tid; e < 512; e += nthreads) {
            const int p = e >> 8, b = e & 255;
            const uint32_t unit = p == 0 ? 0x22u : 0x44u, base = p == 0 ? 0x10101010u : 0u;
            uint32_t lo = base, hi = base;
            for (int c = 0; c < 4; ++c) {
                if (b >> c & 1) lo += unit << (8 * c);
                if (b >> (4 + c) & 1) hi += unit << (8 * c);
            }
            t[e] = make_uint2(lo, hi);
        }
    } else if constexpr (Q == 3) {
        uint32_t *t = (uint32_t *)tab;                 // [plane][256]
        for (int e = tid; e < 768; e += nthreads) {
            const int p = e >> 8, b = e & 255;
            uint32_t w = 0u;
            for (int c = 0; c < 8; ++c)
                if (b >> c & 1) w |= 1u << (4 * c + p);
            t[e] = w;
        }
    }
}
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// the values a weight of one group can take, as prmt sources
template <int Q>
struct GroupValues {
    uint32_t v[Q == 2 ? 2 : 4];      // q = 2: {v0, v1}, {v2, v3} as fp16 pairs; q = 3: low bytes x2, high bytes x2
};
template <int Q>
__device__ __forceinline__ void group_values(GroupValues<Q> &gv, const uint16_t (&alpha)[Q], uint16_t zero) {
    float val[1 << Q];
    val[0] = __half2float(__ushort_as_half(zero));
#pragma unroll
    for (int p = 0; p < Q; ++p) {
        const float ap = __half2float(__ushort_as_half(alpha[p]));
#pragma unroll
        for (int e = 0; e < (1 << p); ++e) val[(1 << p) + e] = val[e] + ap;
    }
    uint32_t pr[(1 << Q) / 2];
#pragma unroll
    for (int e = 0; e < (1 << Q) / 2; ++e) asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(pr[e]) : "f"(val[2 * e + 1]), "f"(val[2 * e]));
    if constexpr (Q == 2) {
        gv.v[0] = pr[0];
        gv.v[1] = pr[1];
    } else {
        gv.v[0] = prmt_b32(pr[0], pr[1], 0x6420u);     // low bytes of values 0..3
        gv.v[1] = prmt_b32(pr[2], pr[3], 0x6420u);     // 4..7
        gv.v[2] = prmt_b32(pr[0], pr[1], 0x7531u);     // high bytes of values 0..3
        gv.v[3] = prmt_b32(pr[2], pr[3], 0x7531u);     // 4..7
    }
}
// 32 channels (bits[p] = the 32 bits of plane p in channel order) as 16 fp16 pairs
template <int Q>
__device__ __forceinline__ void expand32(const uint32_t (&bits)[Q], const GroupValues<Q> &gv, const unsigned char *tab,
                                         uint32_t (&o)[16]) {
    if constexpr (Q == 2) {
        const uint2 *t = (const uint2 *)tab;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint2 e0 = t[(bits[0] >> (8 * k)) & 0xffu], e1 = t[256 + ((bits[1] >> (8 * k)) & 0xffu)];
            const uint32_t sx = e0.x | e1.x, sy = e0.y | e1.y;
            o[4 * k] = prmt_b32(gv.v[0], gv.v[1], sx);
            o[4 * k + 1] = prmt_b32(gv.v[0], gv.v[1], sx >> 16);
            o[4 * k + 2] = prmt_b32(gv.v[0], gv.v[1], sy);
            o[4 * k + 3] = prmt_b32(gv.v[0], gv.v[1], sy >> 16);
        }
    } else {
        const uint32_t *t = (const uint32_t *)tab;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t code = t[(bits[0] >> (8 * k)) & 0xffu] | t[256 + ((bits[1] >> (8 * k)) & 0xffu)] |
                                  t[512 + ((bits[2] >> (8 * k)) & 0xffu)];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t sel = h ? code >> 16 : code;
                const uint32_t lb = prmt_b32(gv.v[0], gv.v[1], sel), hb = prmt_b32(gv.v[2], gv.v[3], sel);
                o[4 * k + 2 * h] = prmt_b32(lb, hb, 0x5140u);
                o[4 * k + 2 * h + 1] = prmt_b32(lb, hb, 0x7362u);
            }
        }
    }
}

// What a dequantizer thread fetches for one slice of 512 channels: the 16 bytes per plane that hold
// the 128 channels of its row in its quarter of the slice, and the fp16 scales / zero of the
// (up to four) groups they fall into, low bits first.
template <int Q>
struct RawSlice {
    uint4 w[Q];
    uint2 mt[Q + 1];
};
// ln = lane of the streaming layout (4 r + quarter)
template <int Q>
__device__ __forceinline__ void load_slice(RawSlice<Q> &rw, const GemmArgs &a, int sl, int oct, int ln, bool row_ok) {
#pragma unroll
    for (int p = 0; p < Q; ++p) {
        rw.w[p] = make_uint4(0u, 0u, 0u, 0u);
        if (row_ok)
            rw.w[p] = __ldg((const uint4 *)(a.planes + (((int64_t)sl * a.octs + oct) * Q + p) * kCellBytes + ln * 16));
    }
#pragma unroll
    for (int p = 0; p <= Q; ++p) {
        const uint16_t *mp = a.meta + (((((int64_t)sl * a.duos + (oct >> 1)) * (Q + 1) + p) * 32 + ln) * 2 + (oct & 1)) * a.gpw;
        rw.mt[p] = make_uint2(0u, 0u);
        if (row_ok) {
            if (a.gpw == 4) rw.mt[p] = __ldg((const uint2 *)mp);
            else if (a.gpw == 2) rw.mt[p].x = __ldg((const uint32_t *)mp);
            else rw.mt[p].x = __ldg(mp);
        }
    }
}
// the four words of a plane in source order: byte pair s of the lane's 16 bytes is stored at s ^ r
__device__ __forceinline__ void source_words(const uint4 &w, int r, uint32_t (&o)[4]) {
    uint32_t w0 = w.x, w1 = w.y, w2 = w.z, w3 = w.w, t;
    if (r & 2) { t = w0; w0 = w1; w1 = t; t = w2; w2 = w3; w3 = t; }
    if (r & 4) { t = w0; w0 = w2; w2 = t; t = w1; w1 = w3; w3 = t; }
    if (r & 1) {
        w0 = __funnelshift_l(w0, w0, 16); w1 = __funnelshift_l(w1, w1, 16);
        w2 = __funnelshift_l(w2, w2, 16); w3 = __funnelshift_l(w3, w3, 16);
    }
    o[0] = w0; o[1] = w1; o[2] = w2; o[3] = w3;
}

template <int Q>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
dequant_gemm_pair_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap xmap) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const uint32_t tiles = (sbase + 1023u) & ~1023u;          // operand tiles need 1024-byte alignment
    unsigned char *tiles_ptr = smem_raw + (tiles - sbase);
    const uint32_t lut_u32 = tiles + kPairStages * kPairXStage;
    uint2 *lut = (uint2 *)(tiles_ptr + kPairStages * kPairXStage);
    uint32_t *sel_lut = (uint32_t *)(tiles_ptr + kPairStages * kPairXStage + 128);   // 2 x 16 words
    const unsigned char *byte_tab = tiles_ptr + kPairStages * kPairXStage + 256;   // kByteTableBytes
    const uint32_t bars = lut_u32 + kLutBytes;
    // barriers: full[s] and acc_empty (waited for in CTA 0 only), empty[s], acc_full; TMEM base; flag.
    // full[s] counts both operands of a K step: the token tile's bytes of both CTAs (announced by
    // CTA 0's producer) and one arrival per dequantizer warp that wrote its rows, so that the
    // issuing thread waits once per step.
    const uint32_t bar_full = bars, bar_empty = bars + 8 * kPairStages;
    const uint32_t bar_acc = bars + 16 * kPairStages, bar_acc_empty = bar_acc + 8, bar_turn = bar_acc + 16;
    uint32_t *tmem_slot = (uint32_t *)(tiles_ptr + kPairStages * kPairXStage + kLutBytes + 16 * kPairStages + 32);
    volatile int *fail = (volatile int *)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_rank();                     // 0: issues the products
    const int pair = (int)(blockIdx.x >> 1), npairs = (int)(gridDim.x >> 1);
    const int half_m = a.tile_m >> 1;                         // tokens this CTA brings in
    const int ksteps = a.kp / kPairStepK;                     // a multiple of 4: the streaming layout pads K to 512
    const int tok_tiles = (a.m + a.tile_m - 1) / a.tile_m;
    const int row_tiles = (a.n + 255) / 256;
    const int ntiles = row_tiles * tok_tiles;
    // Order of the tiles = (256 rows) x (tile_m tokens): the token tiles go in groups of a.tok_group
    // whose activations stay in L2 together; inside a group the row tiles in turn, and for a row
    // tile the group's token tiles one after the other (so its packed weights come from HBM once
    // per group, and the activations once per group instead of once per row tile).
    const int group_tiles = row_tiles * a.tok_group;
    auto row_tile_of = [&](int tile) {
        const int grp = tile / group_tiles, rem = tile - grp * group_tiles;
        const int width = min(a.tok_group, tok_tiles - grp * a.tok_group);
        return rem / width;
    };
    // Few tiles (few tokens, few rows): K is split S ways so that all pairs have work.  A unit is
    // (tile, part of K) = S consecutive unit numbers per tile; its sums go to slab number `part`
    // of S fp32 slabs [m][n] in the workspace (a.acc), which a small kernel adds up and finishes.
    const int S = a.ksplit, slices_total = ksteps >> 2;
    const int nunits = ntiles * S;
    auto unit_tile = [&](int u) { return u / S; };
    auto unit_s0 = [&](int u) { return slices_total * (u % S) / S; };
    auto unit_s1 = [&](int u) { return slices_total * (u % S + 1) / S; };
    auto tok_tile_of = [&](int tile) {
        const int grp = tile / group_tiles, rem = tile - grp * group_tiles;
        const int width = min(a.tok_group, tok_tiles - grp * a.tok_group);
        return grp * a.tok_group + rem % width;
    };

    if (tid == 0) {
        for (int s = 0; s < kPairStages; ++s) {
            mbar_init(bar_full + 8 * s, 1 + 2 * 4);             // producer of CTA 0; the four warps of the step, both CTAs
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 2);                                  // both issuing threads
        mbar_init(bar_turn, 1);
        mbar_init(bar_turn + 8, 1);
        mbar_init(bar_acc_empty, 2 * kPairDeqWarps);            // every epilogue warp of both CTAs
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *fail = 0;
    }
    if (tid < 16) fill_dequant_tables(tid, lut, sel_lut);
    if constexpr (Q == 2 || Q == 3) fill_byte_tables<Q>(tid, kPairThreads, tiles_ptr + kPairStages * kPairXStage + 256);
    if (warp == 1) {   // all of tensor memory, in both CTAs with one instruction each
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kPairTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // the peer's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // barriers of CTA 0 as seen from here
    const uint32_t lead_full = map_to_cta(bar_full, 0);
    const uint32_t lead_acc_empty = map_to_cta(bar_acc_empty, 0);

    // The pair walks its tiles pair, pair + npairs, ...; K steps are counted over all of them (g), so
    // the ring of four stages and the barrier phases run on across tile boundaries: while the
    // accumulator of a tile is read back, the operands of the next tile's first K steps are
    // already being made.
    if (warp == 0) {
        // ------------------------------ TMA producer --------------------------------------
        if (lane == 0) {
            const uint32_t xbytes = (uint32_t)a.tile_m * kPairStepK * 2;  // both halves, both boxes
            int g = 0;
            bool ok = true;
            for (int u = pair; u < nunits && ok; u += npairs) {
                const int m0 = tok_tile_of(unit_tile(u)) * a.tile_m;
                for (int kt = 4 * unit_s0(u); kt < 4 * unit_s1(u); ++kt, ++g) {
                    const int s = g % kPairStages;
                    if (g >= kPairStages) ok = pair_wait(bar_empty + 8 * s, ((g / kPairStages) - 1) & 1, fail);
                    if (!ok) break;
                    if (rank == 0) mbar_expect_tx(bar_full + 8 * s, xbytes);
#pragma unroll
                    for (int bx = 0; bx < 2; ++bx)
                        tma_load_2d_pair(tiles + s * kPairXStage + bx * kPairXBox, &xmap, kt * kPairStepK + bx * kTileK,
                                         m0 + (int)rank * half_m, lead_full + 8 * s);
                }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // ------------------------------ MMA issuers ---------------------------------------
        // Two threads of CTA 0 take the K steps in turn (warp 1 the even ones, warp 2 the odd ones):
        // the tensor cores take a product only when the one before has started, so a single thread
        // spends a step's whole time issuing, and its waits and commits between two steps leave
        // the pipe idle; with two threads one waits and commits while the other issues.  They hand
        // the turn to each other (bar_turn), so the products are issued in the order of the K steps
        // and the sums come out the same in every run.
        if (lane == 0 && rank == 0) {
            const int who = warp - 1;
            const uint32_t idesc = pair_idesc(a.tile_m);
            const uint32_t peer_empty = map_to_cta(bar_empty, 1), peer_acc = map_to_cta(bar_acc, 1);
            int it = 0, mine = 0, g0 = 0;         // units; steps this thread has issued; steps of the units before
            bool ok = true;
            for (int u = pair; u < nunits && ok; u += npairs, ++it) {
                const int kt0 = 4 * unit_s0(u), kt1 = 4 * unit_s1(u);
                // the accumulator of the tile before has been read back by both CTAs
                if (who == 0 && it >= 1) ok = pair_wait(bar_acc_empty, (uint32_t)(it - 1) & 1u, fail);
                if (!ok) break;
                for (int kt = kt0 + who; kt < kt1; kt += 2, ++mine) {
                    const int g = g0 + kt - kt0;
                    const int s = g % kPairStages;
                    const uint32_t ph = (g / kPairStages) & 1;
                    ok = pair_wait(bar_full + 8 * s, ph, fail);
                    // my turn: the other thread has issued the step before
                    if (ok && (who == 1 || mine >= 1))
                        ok = pair_wait(bar_turn + 8 * who, (uint32_t)(who == 1 ? mine : mine - 1) & 1u, fail);
                    if (!ok) break;
                    tc_fence_after();
                    const uint64_t bdesc = umma_desc(tiles + s * kPairXStage);
                    const uint32_t acol = tmem_base + kPairAccCols + (uint32_t)s * kPairACols;
#pragma unroll
                    for (int kk = 0; kk < kPairStepK / 16; ++kk)    // 16 channels = 8 columns of A, 32 bytes of B
                        umma_f16_ts_pair(tmem_base, acol + 8 * kk, bdesc + (uint64_t)((kk >> 2) * (kPairXBox >> 4) + 2 * (kk & 3)),
                                         idesc, (kt > kt0 || kk > 0) ? 1u : 0u);
                    tc_fence_before();
                    mbar_arrive(bar_turn + 8 * (who ^ 1));
                    umma_commit_pair(bar_empty + 8 * s);           // the stage is free again, in both CTAs
                    umma_commit_pair(peer_empty + 8 * s);
                }
                // also after a wait that gave up: the products issued so far end, both CTAs' epilogues wake
                umma_commit_pair(bar_acc);
                umma_commit_pair(peer_acc);
                g0 += kt1 - kt0;
            }
        }
    } else if (warp >= 4) {
        // ------------------------------ dequantizers --------------------------------------
        const int wd = warp - 4;
        const int q4 = warp & 3;                 // lanes 32 q4 .. +31 of tensor memory belong to this warp
        const int part = wd >> 2;                // quarter of every slice = K step `part` of its four = stage `part`
        const int t = 32 * q4 + lane;            // weight row inside this CTA's half of the tile
        const uint32_t tlane = tmem_base + ((uint32_t)(32 * q4) << 16);

        // the accumulator of a finished tile: read back, + bias, stored as y[token][row]
        auto epilogue = [&](int unit, uint32_t parity) {
            const int tile = unit_tile(unit), ks = unit % S;
            const int row = row_tile_of(tile) * 256 + 128 * (int)rank + t;
            const int m0 = tok_tile_of(tile) * a.tile_m;
            pair_wait(bar_acc, parity, fail);
            tc_fence_after();
            float bv = 0.f;
            if (a.bias && row < a.n) bv = __half2float(__ushort_as_half(a.bias[row]));
            const bool good = row < a.n && !*fail;
            // tells CTA 0 that this warp has read its part: the next tile's products may overwrite it
            auto release = [&]() {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lead_acc_empty);
            };
            // This warp's columns are at most two chunks of 32.  The accumulator is handed back as soon
            // as the second chunk is in registers; for 16-bit outputs the first chunk waits there as
            // finished, packed values, so that nothing is stored before the hand-back.
            const int c00 = 32 * part, c01 = c00 + 32 * (kPairDeqWarps / 4);
            uint32_t v[32];
            auto load32 = [&](int c0) {
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                      "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
                      "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
                      "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(tlane + (uint32_t)c0) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            };
            auto store32 = [&](int c0) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int tok = m0 + c0 + c;
                    if (tok < a.m) {
                        const float o = __uint_as_float(v[c]) + bv;
                        const int64_t idx = (int64_t)tok * a.n + row;
                        if (S > 1) a.acc[(int64_t)ks * a.m * a.n + idx] = __uint_as_float(v[c]);   // this part's slab; the finishing kernel adds them up
                        else if (a.y_dtype == HLQ_F16) ((__half *)a.y)[idx] = __float2half_rn(o);
                        else if (a.y_dtype == HLQ_BF16) ((__nv_bfloat16 *)a.y)[idx] = __float2bfloat16_rn(o);
                        else ((float *)a.y)[idx] = o;
                    }
                }
            };
            if (c00 >= a.tile_m) {                       // a narrow tile leaves this warp nothing
                release();
            } else if (c01 >= a.tile_m) {                // one chunk
                load32(c00);
                release();
                if (good) store32(c00);
            } else if (a.y_dtype == HLQ_F32 || S > 1) {  // two chunks of fp32 values: no room to keep the first
                load32(c00);
                if (good) store32(c00);
                load32(c01);
                release();
                if (good) store32(c01);
            } else {
                load32(c00);
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float lo = __uint_as_float(v[2 * i]) + bv, hi = __uint_as_float(v[2 * i + 1]) + bv;
                    if (a.y_dtype == HLQ_F16) {
                        const __half2 h2 = __floats2half2_rn(lo, hi);
                        pk[i] = *(const uint32_t *)&h2;
                    } else {
                        const __nv_bfloat162 b2 = __floats2bfloat162_rn(lo, hi);
                        pk[i] = *(const uint32_t *)&b2;
                    }
                }
                load32(c01);
                release();
                if (good) {
                    store32(c01);
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const int tok = m0 + c00 + c;
                        if (tok < a.m) ((uint16_t *)a.y)[(int64_t)tok * a.n + row] = (uint16_t)(pk[c >> 1] >> (16 * (c & 1)));
                    }
                }
            }
        };

        RawSlice<Q> cur, nxt;
        auto row_of_unit = [&](int u) { return (u < nunits ? row_tile_of(unit_tile(u)) : 0) * 256 + 128 * (int)rank + t; };
        int n = row_of_unit(pair);
        if (pair < nunits) load_slice<Q>(cur, a, unit_s0(pair), n >> 3, 4 * (n & 7) + part, n < a.np);
        int gs = 0, it = 0;                      // slices and units so far
        int pending = -1;                        // unit whose accumulator is still to be read back
        bool ok = true;
        for (int u = pair; u < nunits && ok; u += npairs, ++it) {
            const int r = n & 7;
            const int gsel = r >> a.gshift;      // stored group u holds source group u ^ gsel
            const int sl0 = unit_s0(u), sl1 = unit_s1(u);
            for (int sl = sl0; sl < sl1 && ok; ++sl, ++gs) {
                // the next slice of this unit, else the first slice of the next unit
                {
                    int nn = n, nsl = sl + 1;
                    if (nsl == sl1) {
                        nsl = u + npairs < nunits ? unit_s0(u + npairs) : 0;
                        nn = row_of_unit(u + npairs);
                    }
                    if (sl + 1 < sl1 || u + npairs < nunits) load_slice<Q>(nxt, a, nsl, nn >> 3, 4 * (nn & 7) + part, nn < a.np);
                }
                uint32_t src[Q][4];
#pragma unroll
                for (int p = 0; p < Q; ++p) source_words(cur.w[p], r, src[p]);
                // K step 4 gs + part lives in stage `part`: the ring is one slice deep.  Half of the
                // weights are made before the wait for the stage (it is busy for as long as the products
                // that read it, and the arithmetic need not wait for them), the other half after.
                const int s = part;
                GroupValues<(Q == 2 || Q == 3) ? Q : 2> gv;
                auto make = [&](int ws, uint32_t (&o)[16]) {                  // 32 channels of the lane's 128
                    const int u = ((ws * a.gpw) >> 2) ^ gsel;
                    uint32_t bits[Q];
#pragma unroll
                    for (int p = 0; p < Q; ++p) bits[p] = src[p][ws];
                    // scales and zero of the group: anew only where the group changes (g = 128: once
                    // per slice, g = 64: twice, g = 32: for every 32 channels)
                    const bool fresh = ws == 0 || a.gpw == 4 || (a.gpw == 2 && ws == 2);
                    uint16_t al[Q], z = 0;
                    if (fresh || !(Q == 2 || Q == 3)) {
#pragma unroll
                        for (int p = 0; p < Q; ++p)
                            al[p] = (uint16_t)((((uint64_t)cur.mt[p].y << 32 | cur.mt[p].x) >> (16 * u)) & 0xffffu);
                        z = (uint16_t)((((uint64_t)cur.mt[Q].y << 32 | cur.mt[Q].x) >> (16 * u)) & 0xffffu);
                    }
                    if constexpr (Q == 2 || Q == 3) {
                        if (fresh) group_values<Q>(gv, al, z);
                        expand32<Q>(bits, gv, byte_tab, o);
                    } else {
                        dequant_channels<Q, 32>(bits, al, z, lut, sel_lut, o);
                    }
                };
                auto put = [&](int ws, const uint32_t (&o)[16]) {
                    asm volatile(
                        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                        ::"r"(tlane + kPairAccCols + (uint32_t)s * kPairACols + (uint32_t)(16 * ws)), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                          "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7]), "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]),
                          "r"(o[12]), "r"(o[13]), "r"(o[14]), "r"(o[15]) : "memory");
                };
                {
                    uint32_t o0[16], o1[16];
                    make(0, o0);
                    make(1, o1);
                    if (gs >= 1) ok = pair_wait(bar_empty + 8 * s, (uint32_t)(gs - 1) & 1u, fail);
                    if (!ok) break;
                    tc_fence_after();
                    put(0, o0);
                    put(1, o1);
                }
                {
                    uint32_t o2[16], o3[16];
                    make(2, o2);
                    put(2, o2);
                    make(3, o3);
                    put(3, o3);
                }
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(lead_full + 8 * s);
                cur = nxt;
                // the tile before: its accumulator is read back once this tile's first operands are on
                // their way, so that the tensor cores wait for the read-back alone
                if (sl == sl0 && pending >= 0 && ok) {
                    epilogue(pending, (uint32_t)(it - 1) & 1u);
                    pending = -1;
                }
            }
            pending = u;
            n = row_of_unit(u + npairs);
        }
        if (pending >= 0) epilogue(pending, (uint32_t)(it - 1) & 1u);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();            // nothing of the peer still arrives here or reads this CTA's operands
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kPairTmemCols)
                     : "memory");
    }
    if (tid == 0 && *fail) atomicExch(a.status, 1);
}

// Finishes a launch whose K was split: y = sum of the parts' slabs (+ bias) in the output type.
// The parts are added in their order, so the result is the same in every run.
__global__ void pair_finish_kernel(const float *__restrict__ acc, void *__restrict__ y, const uint16_t *__restrict__ bias,
                                   long long total, int n, int parts, int y_dtype) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float o = 0.f;
        for (int p = 0; p < parts; ++p) o += __ldcs(acc + (long long)p * total + i);
        if (bias) o += __half2float(__ushort_as_half(bias[i % n]));
        if (y_dtype == HLQ_F16) ((__half *)y)[i] = __float2half_rn(o);
        else if (y_dtype == HLQ_BF16) ((__nv_bfloat16 *)y)[i] = __float2bfloat16_rn(o);
        else ((float *)y)[i] = o;
    }
}

// How many parts to split K into, by a cost in microseconds fitted to measurements on a B200: a
// slice of 512 channels takes a pair about 1.8, a unit's first operands and its read-back 8, the
// finishing kernel 4 plus its reads at 4 bytes per part and output.  At most max_parts slabs fit.
int choose_ksplit(int ntiles, int slices, int pairs, long long outputs, int max_parts) {
    int best_s = 1;
    double best = -1.0;
    for (int sp = 1; sp <= slices && sp <= max_parts && sp <= 16; ++sp) {
        const long long rounds = ((long long)ntiles * sp + pairs - 1) / pairs;
        const double unit = 1.8 * ((slices + sp - 1) / sp) + 8.0;
        const double cost = rounds * unit + (sp > 1 ? 4.0 + 4.0e-6 * sp * outputs / 4.0 : 0.0);
        if (best < 0 || cost < best * 0.97) {      // a split must win clearly
            best = cost;
            best_s = sp;
        }
    }
    return best_s;
}

template <int Q>
int launch_pair_inst(GemmArgs &a, const CUtensorMap &xmap, int ntiles, size_t acc_bytes, cudaStream_t stream) {
    static int pairs_cached[64] = {};        // clusters of two that run at once, per device; 0 = not asked yet
    int dev = 0;
    HLQ_CUDA(cudaGetDevice(&dev));
    auto kernel = dequant_gemm_pair_kernel<Q>;
    int &pairs = pairs_cached[dev & 63];
    if (pairs == 0) {
        HLQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kPairDynSmem));
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 1024);
        cfg.blockDim = dim3(kPairThreads);
        cfg.dynamicSmemBytes = kPairDynSmem;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int nclusters = 0;
        HLQ_CUDA(cudaOccupancyMaxActiveClusters(&nclusters, kernel, &cfg));
        if (nclusters < 1) return HLQ_ERR_UNSUPPORTED;
        pairs = nclusters;
    }
    // few tiles: split K, if the workspace has room for the fp32 sums
    a.ksplit = 1;
    const long long total = (long long)a.m * a.n;
    if (ntiles < pairs && a.acc && acc_bytes >= 2 * (size_t)total * sizeof(float))
        a.ksplit = choose_ksplit(ntiles, a.kp / 512, pairs, total, (int)(acc_bytes / ((size_t)total * sizeof(float))));
    const int nunits = ntiles * a.ksplit;
    const int use = nunits < pairs ? nunits : pairs;
    kernel<<<2 * use, kPairThreads, kPairDynSmem, stream>>>(a, xmap);
    count_launch();
    int rc = note_cuda(cudaGetLastError());
    if (rc || a.ksplit == 1) return rc;
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    pair_finish_kernel<<<(int)blocks, 256, 0, stream>>>(a.acc, a.y, a.bias, total, a.n, a.ksplit, a.y_dtype);
    count_launch();
    return note_cuda(cudaGetLastError());
}

}  // namespace

// Tokens per pair tile: a multiple of 32 from 128 to 256 that wastes the fewest waves of SM pairs.
int pair_tile_tokens(int n, int m, int sms, double *cost) {
    const int pairs = sms / 2 > 0 ? sms / 2 : 1;
    double best = 1e300;
    int tile = 256;
    const int lo = m >= 128 ? 128 : ((m + 31) / 32 * 32);
    for (int tm = 256; tm >= lo; tm -= 32) {
        const long long tiles = (long long)((n + 255) / 256) * ((m + tm - 1) / tm);
        const long long waves = (tiles + pairs - 1) / pairs;
        const double c = (double)waves * tm;
        if (c < best * 0.999) {
            best = c;
            tile = tm;
        }
    }
    if (cost) *cost = best;
    return tile;
}

int launch_dequant_gemm_pair(const GemmArgs &a_in, int q, const void *x, int sms, float *acc, size_t acc_bytes,
                             cudaStream_t stream) {
    if (a_in.m < 1 || sms < 2) return HLQ_ERR_UNSUPPORTED;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return HLQ_ERR_NO_DEVICE;
    GemmArgs a = a_in;
    a.acc = acc;
    a.tile_m = pair_tile_tokens(a.n, a.m, sms, nullptr);
    {
        // token tiles whose activations (tile_m x k fp16 each) fit a third of a B200's L2 together
        const long long tile_bytes = (long long)a.tile_m * a.k * 2, budget = 40ll << 20;
        const int tok_tiles = (a.m + a.tile_m - 1) / a.tile_m;
        long long g = budget / (tile_bytes > 0 ? tile_bytes : 1);
        a.tok_group = (int)(g < 1 ? 1 : (g > tok_tiles ? tok_tiles : g));
    }
    CUtensorMap xmap;
    const cuuint64_t dims[2] = {(cuuint64_t)a.k, (cuuint64_t)a.m};
    const cuuint64_t strides[1] = {(cuuint64_t)a.k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)(a.tile_m / 2)};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return HLQ_ERR_INVALID_ARGUMENT;
    const int ntiles = ((a.n + 255) / 256) * ((a.m + a.tile_m - 1) / a.tile_m);
    switch (q) {
        case 1: return launch_pair_inst<1>(a, xmap, ntiles, acc_bytes, stream);
        case 2: return launch_pair_inst<2>(a, xmap, ntiles, acc_bytes, stream);
        case 3: return launch_pair_inst<3>(a, xmap, ntiles, acc_bytes, stream);
        case 4: return launch_pair_inst<4>(a, xmap, ntiles, acc_bytes, stream);
    }
    return HLQ_ERR_SHAPE;
}

}  // namespace gemm
}  // namespace hlq
