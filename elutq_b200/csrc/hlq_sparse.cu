// The runtime's optional extra bit-plane ("sparse" weights): for a list of blocks of 32 output
// rows x one group of input channels, one more bit-plane with one fp16 scale per row,
//     w[x + r, y + c] += scale[pair][r] * bit[pair][r][c].
//
// Replaces, for the GPU path:
//   C++/ops/src/arm/parameters.cpp:44-64           loader (weight_mask.bin, the tails of w_quant.bin / w_scale.bin)
//   C++/ops/src/arm/arm_t_mac_kernal.cpp:554-646   re-layout of the blocks
//   C++/ops/src/arm/arm_t_mac_kernal.cpp:678-788   the kernel (table lookups per block, scale, add into out)
//   C++/ops/src/arm/arm_gemm.cpp:390-563           its drivers
// The blocks are few and small next to the dense planes, so they keep their exported order on
// the device ([pair][32 rows][g/8 bytes], scales [pair][32]) and one warp handles one block: a
// lane owns a row, the group's activations sit in shared memory, and the row's sum goes into
// the fp32 accumulators of the LUT GEMV BEFORE that kernel runs (its completion pass then writes
// dense + extra plane with one rounding), or is added to y after the other kernels.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <new>
#include <vector>

#include "hlq_internal.h"

namespace hlq {

constexpr int kSparseWarps = 4;      // blocks (pairs) per CTA
constexpr int kSparseMaxG = 1024;    // activations of one group held per warp

struct SparseArgs {
    const uint32_t *mask;     // [pairs][2], coordinates of this shard
    const uint8_t *blocks;    // [pairs][32][g/8]
    const uint16_t *scales;   // [pairs][32]
    const void *x;            // [m][k]
    float *acc;               // pre-add: fp32 [m][acc_stride]; else nullptr
    void *y;                  // post-add: [m][n] of y_dtype
    int pairs, m, k, n, g, acc_stride;
    int x_dtype, y_dtype;
};

__global__ void __launch_bounds__(kSparseWarps * 32) sparse_plane_kernel(const SparseArgs a) {
    __shared__ float xs[kSparseWarps][kSparseMaxG];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = blockIdx.x * kSparseWarps + warp;
    if (p >= a.pairs) return;
    // A warp takes a whole run of consecutive pairs with the same first row (the list is sorted by
    // rows, parameters.cpp hands it over that way and the reference's kernel relies on it too,
    // arm_t_mac_kernal.cpp:766-785): their sums meet in a register and the output row is touched
    // once.  Pairs in the middle of a run are left to the warp of the run's first pair; the final
    // additions are atomic, so an unsorted list costs precision of 16-bit outputs, not correctness.
    const int x0 = (int)a.mask[2 * p];
    if (p > 0 && (int)a.mask[2 * (p - 1)] == x0) return;
    int pend = p + 1;
    while (pend < a.pairs && (int)a.mask[2 * pend] == x0) ++pend;
    const int gb = a.g / 8;
    const int row = x0 + lane;
    for (int mi = 0; mi < a.m; ++mi) {
        float total = 0.f;
        for (int pp = p; pp < pend; ++pp) {
            const int y0 = (int)a.mask[2 * pp + 1];
            const uint8_t *bits = a.blocks + ((size_t)pp * 32 + lane) * gb;
            const float scale = __half2float(__ushort_as_half(a.scales[(size_t)pp * 32 + lane]));
            const uint16_t *xr = (const uint16_t *)a.x + (size_t)mi * a.k + y0;
            for (int c = lane; c < a.g; c += 32)
                xs[warp][c] = a.x_dtype == HLQ_BF16 ? __uint_as_float((uint32_t)xr[c] << 16)
                                                    : __half2float(__ushort_as_half(xr[c]));
            __syncwarp();
            float s = 0.f;
            for (int i = 0; i < gb; ++i) {
                const unsigned b = bits[i];
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if ((b >> j) & 1u) s += xs[warp][8 * i + j];
            }
            total += s * scale;
            __syncwarp();
        }
        if (row < a.n) {
            if (a.acc) {
                atomicAdd(a.acc + (size_t)mi * a.acc_stride + row, total);
            } else {
                const size_t idx = (size_t)mi * a.n + row;
                if (a.y_dtype == HLQ_F32) atomicAdd((float *)a.y + idx, total);
                else if (a.y_dtype == HLQ_F16) atomicAdd((__half *)a.y + idx, __float2half_rn(total));
                else atomicAdd((__nv_bfloat16 *)a.y + idx, __float2bfloat16_rn(total));
            }
        }
    }
}

// acc != nullptr: add into fp32 accumulators [m][acc_stride]; else read-modify-write y.
int launch_sparse_plane(const hlq_weight *w, int m, const void *x, int x_dtype, float *acc, int acc_stride, void *y,
                        int y_dtype, cudaStream_t stream) {
    if (!w->sp_pairs) return HLQ_OK;
    SparseArgs a;
    a.mask = w->d_sp_mask;
    a.blocks = w->d_sp_blocks;
    a.scales = w->d_sp_scales;
    a.x = x;
    a.acc = acc;
    a.y = y;
    a.pairs = w->sp_pairs; a.m = m; a.k = w->k; a.n = w->n; a.g = w->g; a.acc_stride = acc_stride;
    a.x_dtype = x_dtype; a.y_dtype = y_dtype;
    const int grid = (w->sp_pairs + kSparseWarps - 1) / kSparseWarps;
    sparse_plane_kernel<<<grid, kSparseWarps * 32, 0, stream>>>(a);
    HLQ_CUDA(cudaGetLastError());
    count_launch();
    return HLQ_OK;
}

void free_sparse(hlq_weight *w) {
    if (w->d_sp_mask) cudaFree(w->d_sp_mask);
    if (w->d_sp_blocks) cudaFree(w->d_sp_blocks);
    if (w->d_sp_scales) cudaFree(w->d_sp_scales);
    w->d_sp_mask = nullptr;
    w->d_sp_blocks = nullptr;
    w->d_sp_scales = nullptr;
    w->sp_pairs = 0;
}

}  // namespace hlq

using namespace hlq;

extern "C" {

int hlq_weight_set_sparse(hlq_weight *w, const uint32_t *h_mask, int pairs, const uint8_t *h_blocks,
                          const uint16_t *h_scales, void *stream_) {
    if (!w || pairs < 0 || (pairs && (!h_mask || !h_blocks || !h_scales))) return HLQ_ERR_INVALID_ARGUMENT;
    if (w->g > kSparseMaxG) return HLQ_ERR_UNSUPPORTED;
    cudaStream_t stream = (cudaStream_t)stream_;
    const int g = w->g, gb = g / 8;
    // keep the blocks of this shard, in the shard's coordinates
    std::vector<uint32_t> mask;
    std::vector<uint8_t> blocks;
    std::vector<uint16_t> scales;
    for (int p = 0; p < pairs; ++p) {
        const long long x = h_mask[2 * p], y = h_mask[2 * p + 1];
        if (x % 32 || y % g || x + 32 > (long long)w->n_full + 31 || y + g > w->k_full) return HLQ_ERR_SHAPE;
        if (x < w->n0 || x >= (long long)w->n0 + w->n || y < w->k0 || y >= (long long)w->k0 + w->k) continue;
        mask.push_back((uint32_t)(x - w->n0));
        mask.push_back((uint32_t)(y - w->k0));
        blocks.insert(blocks.end(), h_blocks + (size_t)p * 32 * gb, h_blocks + (size_t)(p + 1) * 32 * gb);
        scales.insert(scales.end(), h_scales + (size_t)p * 32, h_scales + (size_t)(p + 1) * 32);
    }
    int prev = -1;
    cudaGetDevice(&prev);
    if (cudaSetDevice(w->device) != cudaSuccess) return HLQ_ERR_NO_DEVICE;
    free_sparse(w);
    int rc = HLQ_OK;
    const int kept = (int)(mask.size() / 2);
    if (kept) {
        if (cudaMalloc((void **)&w->d_sp_mask, mask.size() * 4) != cudaSuccess ||
            cudaMalloc((void **)&w->d_sp_blocks, blocks.size()) != cudaSuccess ||
            cudaMalloc((void **)&w->d_sp_scales, scales.size() * 2) != cudaSuccess)
            rc = note_cuda(cudaErrorMemoryAllocation);
        if (!rc) rc = note_cuda(cudaMemcpyAsync(w->d_sp_mask, mask.data(), mask.size() * 4, cudaMemcpyHostToDevice, stream));
        if (!rc) rc = note_cuda(cudaMemcpyAsync(w->d_sp_blocks, blocks.data(), blocks.size(), cudaMemcpyHostToDevice, stream));
        if (!rc) rc = note_cuda(cudaMemcpyAsync(w->d_sp_scales, scales.data(), scales.size() * 2, cudaMemcpyHostToDevice, stream));
        if (!rc) rc = note_cuda(cudaStreamSynchronize(stream));
        if (rc) free_sparse(w);
        else w->sp_pairs = kept;
    }
    if (prev >= 0) cudaSetDevice(prev);
    return rc;
}

int hlq_weight_sparse_pairs(const hlq_weight *w, int *pairs) {
    if (!w || !pairs) return HLQ_ERR_INVALID_ARGUMENT;
    *pairs = w->sp_pairs;
    return HLQ_OK;
}

int hlq_weight_get_sparse(const hlq_weight *w, uint32_t *h_mask, uint8_t *h_blocks, uint16_t *h_scales, void *stream_) {
    if (!w || (w->sp_pairs && (!h_mask || !h_blocks || !h_scales))) return HLQ_ERR_INVALID_ARGUMENT;
    if (!w->sp_pairs) return HLQ_OK;
    cudaStream_t stream = (cudaStream_t)stream_;
    int prev = -1;
    cudaGetDevice(&prev);
    if (cudaSetDevice(w->device) != cudaSuccess) return HLQ_ERR_NO_DEVICE;
    const size_t p = (size_t)w->sp_pairs;
    int rc = note_cuda(cudaMemcpyAsync(h_mask, w->d_sp_mask, p * 8, cudaMemcpyDeviceToHost, stream));
    if (!rc) rc = note_cuda(cudaMemcpyAsync(h_blocks, w->d_sp_blocks, p * 32 * (w->g / 8), cudaMemcpyDeviceToHost, stream));
    if (!rc) rc = note_cuda(cudaMemcpyAsync(h_scales, w->d_sp_scales, p * 64, cudaMemcpyDeviceToHost, stream));
    if (!rc) rc = note_cuda(cudaStreamSynchronize(stream));
    if (prev >= 0) cudaSetDevice(prev);
    return rc;
}

}  // extern "C"
