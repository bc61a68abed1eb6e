// Dequantize + tensor-core GEMM over HLQ weights for prefill (m >= 64), sm_100a.
//
// Replaces the reference's prefill path, which runs one GEMV per token and re-streams all
// weights m times (C++/ops/src/arm/arm_gemm.cpp:362-387).  Here a CTA owns a tile of 128
// output rows x 256 tokens and walks K in steps of 64 channels:
//   warp 0      TMA producer: the 256 x 64 activation tile of every K step, tensor map with
//               128-byte swizzle, mbarrier completion (cp.async.bulk.tensor.2d);
//   warps 4..   dequantizers: two threads per weight row of the tile.  Each reads 4 bytes of
//               each bit-plane from the streaming layout, turns every bit into a 16-bit mask
//               through a 16-entry (nibble) shared-memory table that is free of bank conflicts, forms z + sum_p (mask & alpha_p) in
//               packed fp16 and writes its 64 values as one 128-byte row of the K-major,
//               128-byte-swizzled operand tile; fence.proxy.async + mbarrier arrive;
//   warp 1      MMA issuer: one thread issues four tcgen05.mma (128 x 256 x 16, kind::f16,
//               fp32 accumulator in tensor memory) per K step and commits to the stage's
//               "empty" mbarrier;
//   warps 4..7  epilogue: tcgen05.ld of the 128 x 256 fp32 accumulator (one TMEM lane = one
//               output row), add the bias, store y[token][row].
// D = W_tile . X_tile^T, i.e. the accumulator is y transposed.
//
// Precision: the weights are rounded to fp16 (rel. 2^-11) before the product and
// accumulation is fp32.  kind::f16 wants both operands in one 16-bit format (a descriptor
// with fp16 weights and bf16 activations is an illegal instruction on B200), and bf16 weights
// would carry a rel. 2^-9 rounding, so bf16 activations are first converted to fp16
// (saturating at +-65504) by a small kernel into the workspace.
// All mbarrier waits are bounded; on expiry the CTA sets the status word and carries on to
// its exit so that tensor memory is always released.
#include <cuda.h>

#include <atomic>
#include <cstdlib>

#include "hlq_gemm_dev.cuh"

namespace hlq {
namespace gemm {

template <int ROWS>
struct Cfg {
    static constexpr int kAcc = ROWS / 128;                       // accumulators of 128 rows
    static constexpr int kDeqWarps = ROWS / 16;                   // two threads per weight row
    static constexpr int kThreads = 128 + 32 * kDeqWarps;         // 4 service warps + dequantizers
    static constexpr uint32_t kWBytes = ROWS * kTileK * 2;
    static constexpr uint32_t kStageBytes = kWBytes + kXBytes;
    static constexpr int kStages = ROWS == 128 ? 4 : 3;           // 192 KB of operand tiles either way
    static constexpr uint32_t kDynSmem = 1024 + kStages * kStageBytes + kLutBytes + kBarBytes;
    static constexpr uint32_t kTmemCols = 256 * kAcc;
};

template <int ROWS, int Q>
__global__ void __launch_bounds__(Cfg<ROWS>::kThreads, 1)
dequant_gemm_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap xmap) {
    using C = Cfg<ROWS>;
    constexpr int kStages = C::kStages;
    constexpr uint32_t kStageBytes = C::kStageBytes, kWBytes = C::kWBytes;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const uint32_t sbase = smem_u32(smem_raw);
    const uint32_t tiles = (sbase + 1023u) & ~1023u;          // operand tiles need 1024-byte alignment
    unsigned char *tiles_ptr = smem_raw + (tiles - sbase);
    const uint32_t lut_u32 = tiles + kStages * kStageBytes;
    uint2 *lut = (uint2 *)(tiles_ptr + kStages * kStageBytes);
    uint32_t *sel_lut = (uint32_t *)(tiles_ptr + kStages * kStageBytes + 128);   // 2 x 16 words
    const uint32_t bars = lut_u32 + kLutBytes;
    // barriers: full_x[s], full_w[s], empty[s], acc_full; then the TMEM base and the fail flag
    const uint32_t bar_full_x = bars, bar_full_w = bars + 8 * kStages, bar_empty = bars + 16 * kStages;
    const uint32_t bar_acc = bars + 24 * kStages;
    uint32_t *tmem_slot = (uint32_t *)(tiles_ptr + kStages * kStageBytes + kLutBytes + 24 * kStages + 8);
    int *fail = (int *)(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * ROWS, m0 = blockIdx.y * a.tile_m;
    const int ksteps = a.kp / kTileK;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full_x + 8 * s, 1);
            mbar_init(bar_full_w + 8 * s, C::kDeqWarps);   // one arrival per dequantizer warp
            mbar_init(bar_empty + 8 * s, 1);
        }
        mbar_init(bar_acc, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        *fail = 0;
    }
    if (tid < 16) fill_dequant_tables(tid, lut, sel_lut);
    if (warp == 1) {   // tensor memory: 256 fp32 columns x 128 lanes per accumulator
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(C::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer --------------------------------------
        if (lane == 0) {
            const uint32_t xbytes = (uint32_t)a.tile_m * kTileK * 2;
            for (int kt = 0; kt < ksteps; ++kt) {
                const int s = kt % kStages;
                if (kt >= kStages && !mbar_wait(bar_empty + 8 * s, ((kt / kStages) - 1) & 1)) *fail = 1;
                mbar_expect_tx(bar_full_x + 8 * s, xbytes);
                tma_load_2d(tiles + s * kStageBytes + kWBytes, &xmap, kt * kTileK, m0, bar_full_x + 8 * s);
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ----------------------------------------
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(a.tile_m);
            for (int kt = 0; kt < ksteps; ++kt) {
                const int s = kt % kStages;
                const uint32_t ph = (kt / kStages) & 1;
                if (!mbar_wait(bar_full_x + 8 * s, ph)) *fail = 1;
                if (!mbar_wait(bar_full_w + 8 * s, ph)) *fail = 1;
                tc_fence_after();
                const uint64_t bdesc = umma_desc(tiles + s * kStageBytes + kWBytes);
#pragma unroll
                for (int h = 0; h < C::kAcc; ++h) {
                    const uint64_t adesc = umma_desc(tiles + s * kStageBytes + h * (128 * 128));
#pragma unroll
                    for (int kk = 0; kk < kTileK / 16; ++kk)   // 16 channels = 32 bytes = 2 descriptor units
                        umma_f16(tmem_base + h * 256, adesc + 2 * kk, bdesc + 2 * kk, idesc,
                                 (kt > 0 || kk > 0) ? 1u : 0u);
                }
                umma_commit(bar_empty + 8 * s);
            }
            umma_commit(bar_acc);
        }
    } else if (warp >= 4) {
        // ------------------------------ dequantizers --------------------------------------
        // a warp owns 16 rows; lanes 0-15 take channels 0-31 of the K step, lanes 16-31 channels 32-63
        const int wd = warp - 4;
        const int t = wd * 16 + (lane & 15);     // weight row inside the tile
        const int hh = lane >> 4;
        const int n = n0 + t;
        const bool row_ok = n < a.np;
        const int oct = n >> 3, r = n & 7;
        const bool swap = (r & 1) != 0;          // order of the two byte pairs inside the 4 bytes
        const uint32_t row_smem = (uint32_t)t * 128u;
        Raw<Q> cur, nxt;
        load_raw<Q>(cur, a, 0, oct, r, hh, row_ok);
        for (int kt = 0; kt < ksteps; ++kt) {
            const int s = kt % kStages;
            if (kt + 1 < ksteps) load_raw<Q>(nxt, a, kt + 1, oct, r, hh, row_ok);
            if (kt >= kStages && !mbar_wait(bar_empty + 8 * s, ((kt / kStages) - 1) & 1)) *fail = 1;
            uint32_t bits[Q];                       // the 32 bits of each plane in source order
#pragma unroll
            for (int p = 0; p < Q; ++p) bits[p] = swap ? __funnelshift_l(cur.w[p], cur.w[p], 16) : cur.w[p];
            uint32_t o[16];
            dequant_channels<Q, 32>(bits, cur.al, cur.z, lut, sel_lut, o);
            const uint32_t wrow = tiles + s * kStageBytes + row_smem;
#pragma unroll
            for (int ci = 0; ci < 4; ++ci) {        // 8 channels = one 16-byte chunk, swizzled by the row
                const uint32_t dst = wrow + (uint32_t)(((4 * hh + ci) ^ (t & 7)) << 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(o[4 * ci]), "r"(o[4 * ci + 1]),
                             "r"(o[4 * ci + 2]), "r"(o[4 * ci + 3]) : "memory");
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_full_w + 8 * s);
            cur = nxt;
        }
        // ------------------------------ epilogue ------------------------------------------
        if (!mbar_wait(bar_acc, 0)) *fail = 1;
        tc_fence_after();
        const int q4 = warp & 3;                     // TMEM lanes 32*q4 .. +31 belong to this warp
        const int hacc = (wd >> 2) % C::kAcc;        // accumulator = 128-row half of the tile
        const int cpart = wd / (4 * C::kAcc);        // the warps of one (accumulator, quarter) split the tokens
        const int row = n0 + 128 * hacc + 32 * q4 + lane;
        float bv = 0.f;
        if (a.bias && row < a.n) bv = __half2float(__ushort_as_half(a.bias[row]));
        for (int c0 = 32 * cpart; c0 < a.tile_m; c0 += 64) {
            uint32_t v[32];
            const uint32_t taddr = tmem_base + ((uint32_t)(32 * q4) << 16) + (uint32_t)(hacc * 256 + c0);
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                  "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                  "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
                  "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
                  "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                : "r"(taddr) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < a.n) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int tok = m0 + c0 + c;
                    if (tok < a.m) {
                        const float o = __uint_as_float(v[c]) + bv;
                        const int64_t idx = (int64_t)tok * a.n + row;
                        if (a.y_dtype == HLQ_F16) ((__half *)a.y)[idx] = __float2half_rn(o);
                        else if (a.y_dtype == HLQ_BF16) ((__nv_bfloat16 *)a.y)[idx] = __float2bfloat16_rn(o);
                        else ((float *)a.y)[idx] = o;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::kTmemCols)
                     : "memory");
    }
    if (tid == 0 && *fail) atomicExch(a.status, 1);
}

// bf16 -> fp16, eight values per thread and step, saturating instead of overflowing to inf
__global__ void bf16_to_f16_kernel(const uint4 *__restrict__ in, uint4 *__restrict__ out, int64_t nvec) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
        const uint4 v = in[i];
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float lo = __uint_as_float(w[q] << 16), hi = __uint_as_float(w[q] & 0xffff0000u);
            asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(o[q]) : "f"(hi), "f"(lo));
        }
        out[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

}  // namespace gemm

// 0 or 2 = dequant_gemm_pair_kernel, 1 = dequant_gemm_kernel
static std::atomic<int> g_prefill_kernel{0};

// Tile shape: rows per CTA (128 or 256) and tokens per CTA (multiple of 32 up to 256), chosen
// to waste the fewest SM-waves; ties go to the larger tile (less activation traffic from L2).
static void choose_tiles(int n, int m, int sms, int *rows, int *tile_m) {
    double best = 1e300;
    *rows = 128;
    *tile_m = 256;
    const int tm_min = m >= 128 ? 128 : ((m + 31) / 32 * 32);
    for (int r = 256; r >= 128; r -= 128)
        for (int tm = 256; tm >= tm_min; tm -= 32) {
            const long long tiles = (long long)((n + r - 1) / r) * ((m + tm - 1) / tm);
            const long long waves = (tiles + sms - 1) / sms;
            // 128-row tiles read the activations twice as often per flop: measured ~1.3x slower per flop
            const double cost = (double)waves * r * tm * (r == 128 ? 1.3 : 1.0);
            if (cost < best * 0.999) {
                best = cost;
                *rows = r;
                *tile_m = tm;
            }
        }
}

template <int ROWS, int Q>
static int launch_inst(const gemm::GemmArgs &a, const CUtensorMap &xmap, dim3 grid, cudaStream_t stream) {
    using C = gemm::Cfg<ROWS>;
    static bool configured[64] = {};
    int dev = 0;
    HLQ_CUDA(cudaGetDevice(&dev));
    auto kernel = gemm::dequant_gemm_kernel<ROWS, Q>;
    if (!configured[dev & 63]) {
        HLQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kDynSmem));
        configured[dev & 63] = true;
    }
    kernel<<<grid, C::kThreads, C::kDynSmem, stream>>>(a, xmap);
    count_launch();
    return note_cuda(cudaGetLastError());
}

int launch_dequant_gemm(const hlq_weight *w, int m, const void *x, int x_dtype, void *y, int y_dtype,
                        void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    using namespace gemm;
    if (w->layout != HLQ_LAYOUT_STREAM) return HLQ_ERR_UNSUPPORTED;
    if (x_dtype != HLQ_F16 && x_dtype != HLQ_BF16) return HLQ_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)y & 3)) return HLQ_ERR_ALIGNMENT;
    if (!workspace || workspace_bytes < kWsHeader) return HLQ_ERR_WORKSPACE;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return HLQ_ERR_NO_DEVICE;
    const StreamDims d = stream_dims(w->n, w->k, w->g, w->q);
    if (x_dtype == HLQ_BF16) {
        // fp16 copy of the activations, behind what the LUT kernels keep in the workspace
        const size_t bytes = (size_t)m * w->k * 2, off = gemm_scratch_offset(d);
        if (workspace_bytes < off + bytes) return HLQ_ERR_WORKSPACE;
        void *x16 = (char *)workspace + off;
        const int64_t nvec = (int64_t)(bytes / 16);       // k % 8 == 0
        int64_t blocks = (nvec + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        bf16_to_f16_kernel<<<(int)blocks, 256, 0, stream>>>((const uint4 *)x, (uint4 *)x16, nvec);
        count_launch();
        int rc = note_cuda(cudaGetLastError());
        if (rc) return rc;
        x = x16;
    }
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, w->device);
    GemmArgs a;
    a.planes = w->d_planes;
    a.meta = w->d_meta;
    a.bias = w->d_bias;
    a.y = y;
    a.status = (int *)workspace;
    a.m = m; a.n = w->n; a.k = w->k; a.np = d.np; a.kp = d.kp; a.octs = d.octs; a.duos = d.duos;
    a.gpw = d.gpw; a.gshift = d.gshift;
    a.tile_m = 0;
    a.tok_group = 1;
    a.ksplit = 1;
    a.acc = nullptr;
    a.y_dtype = y_dtype;
    // CTA pairs with the weight operand in tensor memory unless the other kernel is asked for: the
    // pair kernel is the faster one at every number of tokens measured (64 .. 4096)
    const int which = g_prefill_kernel.load(std::memory_order_relaxed);
    if (which != 1) {
        // fp32 sums of a K split (few tokens and few rows): behind the fp16 copy of the tokens
        const size_t acc_off = gemm_acc_offset(m, d);
        float *acc = workspace_bytes > acc_off ? (float *)((char *)workspace + acc_off) : nullptr;
        const int rc = launch_dequant_gemm_pair(a, w->q, x, sms, acc, acc ? workspace_bytes - acc_off : 0, stream);
        if (rc != HLQ_ERR_UNSUPPORTED) return rc;
    }
    int rows = 128, tile_m = 256;
    choose_tiles(w->n, m, sms, &rows, &tile_m);

    CUtensorMap xmap;
    const cuuint64_t dims[2] = {(cuuint64_t)w->k, (cuuint64_t)m};
    const cuuint64_t strides[1] = {(cuuint64_t)w->k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)tile_m};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return HLQ_ERR_INVALID_ARGUMENT;

    a.tile_m = tile_m;
    dim3 grid((w->n + rows - 1) / rows, (m + tile_m - 1) / tile_m);
#define HLQ_GEMM_CASE(R, QV) \
    if (rows == R && w->q == QV) return launch_inst<R, QV>(a, xmap, grid, stream);
    HLQ_GEMM_CASE(128, 1) HLQ_GEMM_CASE(128, 2) HLQ_GEMM_CASE(128, 3) HLQ_GEMM_CASE(128, 4)
    HLQ_GEMM_CASE(256, 1) HLQ_GEMM_CASE(256, 2) HLQ_GEMM_CASE(256, 3) HLQ_GEMM_CASE(256, 4)
#undef HLQ_GEMM_CASE
    return HLQ_ERR_SHAPE;
}

}  // namespace hlq

extern "C" int hlq_select_prefill_kernel(int which) {
    if (which < 0 || which > 2) return HLQ_ERR_INVALID_ARGUMENT;
    hlq::g_prefill_kernel.store(which, std::memory_order_relaxed);
    return HLQ_OK;
}
