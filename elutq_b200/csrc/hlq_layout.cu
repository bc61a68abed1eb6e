// Device kernels for bit-plane packing and for the streaming re-layout.
//
// Replaces, on the GPU:
//   GPTQ/HLQ.py:239-251 (Pack_T_MAC_Weight)                                -> pack / unpack
//   C++/ops/src/arm/arm_t_mac_kernal.cpp:472-552 (load-time weight re-layout) -> repack / unrepack
// All of it is byte and bit movement; results are bit-exact by construction and are checked
// against the host implementations in hlq_host.cpp.
#include "hlq_internal.h"

namespace hlq {

__global__ void pack_bits_kernel(const uint8_t *__restrict__ bits, uint8_t *__restrict__ packed,
                                 int64_t total_bytes) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_bytes; i += stride) {
        const uint2 v = *(const uint2 *)(bits + i * 8);
        // each source byte is 0 or 1: gather the eight low bits
        const uint32_t lo = v.x & 0x01010101u, hi = v.y & 0x01010101u;
        const uint32_t l = (lo | (lo >> 7) | (lo >> 14) | (lo >> 21)) & 0xfu;
        const uint32_t h = (hi | (hi >> 7) | (hi >> 14) | (hi >> 21)) & 0xfu;
        packed[i] = (uint8_t)(l | (h << 4));
    }
}

__global__ void unpack_bits_kernel(const uint8_t *__restrict__ packed, uint8_t *__restrict__ bits,
                                   int64_t total_bytes) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total_bytes; i += stride) {
        const uint32_t b = packed[i];
        uint2 v;
        v.x = (b & 1u) | ((b & 2u) << 7) | ((b & 4u) << 14) | ((b & 8u) << 21);
        v.y = ((b >> 4) & 1u) | ((b & 32u) << 3) | ((b & 64u) << 10) | ((b & 128u) << 17);
        *(uint2 *)(bits + i * 8) = v;
    }
}

// Nearest-combination quantizer of the reference (GPTQ/quant.py:154-174): per element the
// argmin over the 2^q values sum_j s_j * c_j of |value - (w - z)|, first minimum on ties;
// combination c has bit j = (c >> (q - 1 - j)) & 1 (first column slowest, quant.py:12-16).
template <int Q>
__global__ void quantize_with_scales_kernel(const float *__restrict__ w, const float *__restrict__ scales,
                                            const float *__restrict__ zeros, uint8_t *__restrict__ out,
                                            int64_t total, int g) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t b = i / g;
        float s[Q];
#pragma unroll
        for (int j = 0; j < Q; ++j) s[j] = scales[b * Q + j];
        const float t = w[i] - zeros[b];
        float best = INFINITY;
        int arg = 0;
#pragma unroll
        for (int c = 0; c < (1 << Q); ++c) {
            float v = 0.f;
#pragma unroll
            for (int j = 0; j < Q; ++j)
                if ((c >> (Q - 1 - j)) & 1) v = __fadd_rn(v, s[j]);
            const float dist = fabsf(__fsub_rn(v, t));
            if (dist < best) {
                best = dist;
                arg = c;
            }
        }
#pragma unroll
        for (int j = 0; j < Q; ++j) out[i * Q + j] = (uint8_t)((arg >> (Q - 1 - j)) & 1);
    }
}

// one thread per 16-byte lane word of a cell
__global__ void repack_planes_kernel(const uint8_t *__restrict__ w_quant, uint8_t *__restrict__ planes,
                                     StreamDims d) {
    const int64_t words = (int64_t)d.slices * d.octs * d.q * 32;
    const int64_t kb = d.k / 8;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < words; idx += stride) {
        const int lane = (int)(idx & 31);
        int64_t t = idx >> 5;
        const int p = (int)(t % d.q);
        t /= d.q;
        const int oct = (int)(t % d.octs);
        const int s = (int)(t / d.octs);
        const int r = lane >> 2, j = lane & 3;
        const int64_t row = (int64_t)oct * kOctRows + r;
        const int64_t byte0 = (int64_t)s * (kSliceK / 8) + 16 * j;
        uint32_t out[4] = {0, 0, 0, 0};
        if (row < d.n) {
            const uint8_t *src = w_quant + ((int64_t)p * d.n + row) * kb;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const int64_t sb = byte0 + stream_src_byte(i, r);
                const uint32_t v = sb < kb ? src[sb] : 0u;
                out[i >> 2] |= v << (8 * (i & 3));
            }
        }
        *(uint4 *)(planes + idx * 16) = make_uint4(out[0], out[1], out[2], out[3]);
    }
}

__global__ void repack_meta_kernel(const uint16_t *__restrict__ w_scale,
                                   const uint16_t *__restrict__ w_zero, uint16_t *__restrict__ meta,
                                   StreamDims d) {
    const int64_t elems = stream_meta_elems(d);
    const int64_t ng = d.k / d.g;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < elems; idx += stride) {
        int64_t t = idx;
        const int u = (int)(t % d.gpw);
        t /= d.gpw;
        const int ou = (int)(t & 1);
        t >>= 1;
        const int lane = (int)(t & 31);
        t >>= 5;
        const int pp = (int)(t % (d.q + 1));
        t /= (d.q + 1);
        const int oct = (int)(t % d.duos) * 2 + ou;
        const int s = (int)(t / d.duos);
        const int r = lane >> 2, j = lane & 3;
        const int64_t row = (int64_t)oct * kOctRows + r;
        const int64_t grp = ((int64_t)s * kSliceK + 128 * j) / d.g + stream_src_group(d, u, r);
        uint16_t v = 0;
        if (row < d.n && grp < ng)
            v = pp < d.q ? w_scale[((int64_t)pp * d.n + row) * ng + grp] : w_zero[row * ng + grp];
        meta[idx] = v;
    }
}

// one thread per exported byte
__global__ void unrepack_planes_kernel(const uint8_t *__restrict__ planes, uint8_t *__restrict__ w_quant,
                                       StreamDims d) {
    const int64_t kb = d.k / 8;
    const int64_t total = (int64_t)d.q * d.n * kb;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t sb = idx % kb;
        int64_t t = idx / kb;
        const int64_t row = t % d.n;
        const int p = (int)(t / d.n);
        const int oct = (int)(row / kOctRows), r = (int)(row % kOctRows);
        const int s = (int)(sb / (kSliceK / 8));
        const int rem = (int)(sb % (kSliceK / 8));
        const int j = rem / 16, b = rem % 16;
        w_quant[idx] = planes[stream_plane_offset(d, s, oct, p, r * 4 + j, stream_pos_of_src(b, r))];
    }
}

__global__ void unrepack_meta_kernel(const uint16_t *__restrict__ meta, uint16_t *__restrict__ w_scale,
                                     uint16_t *__restrict__ w_zero, StreamDims d) {
    const int64_t ng = d.k / d.g;
    const int64_t total = (int64_t)(d.q + 1) * d.n * ng;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t grp = idx % ng;
        int64_t t = idx / ng;
        const int64_t row = t % d.n;
        const int pp = (int)(t / d.n);
        const int oct = (int)(row / kOctRows), r = (int)(row % kOctRows);
        const int64_t ch = grp * d.g;
        const int s = (int)(ch / kSliceK);
        const int j = (int)((ch % kSliceK) / 128);
        const int su = (int)((ch % 128) / d.g);
        const int u = su ^ (r >> d.gshift);
        const uint16_t v = meta[stream_meta_offset(d, s, oct, pp, r * 4 + j, u)];
        if (pp < d.q) w_scale[((int64_t)pp * d.n + row) * ng + grp] = v;
        else w_zero[row * ng + grp] = v;
    }
}

static int grid_for(int64_t items, int threads) {
    int64_t g = (items + threads - 1) / threads;
    if (g > 148 * 32) g = 148 * 32;
    if (g < 1) g = 1;
    return (int)g;
}

}  // namespace hlq

using namespace hlq;

extern "C" {

int hlq_quantize_with_scales_device(const float *d_w, const float *d_scales, const float *d_zeros, uint8_t *d_out,
                                    int64_t blocks, int g, int q, void *stream) {
    if (blocks < 0 || g <= 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (q < 1 || q > 4) return HLQ_ERR_SHAPE;
    const int64_t total = blocks * g;
    if (total == 0) return HLQ_OK;
    if (!d_w || !d_scales || !d_zeros || !d_out) return HLQ_ERR_INVALID_ARGUMENT;
    const dim3 grid = grid_for(total, 256);
    cudaStream_t st = (cudaStream_t)stream;
    switch (q) {
        case 1: quantize_with_scales_kernel<1><<<grid, 256, 0, st>>>(d_w, d_scales, d_zeros, d_out, total, g); break;
        case 2: quantize_with_scales_kernel<2><<<grid, 256, 0, st>>>(d_w, d_scales, d_zeros, d_out, total, g); break;
        case 3: quantize_with_scales_kernel<3><<<grid, 256, 0, st>>>(d_w, d_scales, d_zeros, d_out, total, g); break;
        default: quantize_with_scales_kernel<4><<<grid, 256, 0, st>>>(d_w, d_scales, d_zeros, d_out, total, g); break;
    }
    count_launch();
    return note_cuda(cudaGetLastError());
}

int hlq_pack_bits_device(const uint8_t *d_bits, uint8_t *d_packed, int q, int64_t n, int64_t k,
                         void *stream) {
    if (q < 0 || n < 0 || k < 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (k % 8) return HLQ_ERR_SHAPE;
    const int64_t total = (int64_t)q * n * (k / 8);
    if (total == 0) return HLQ_OK;
    if (!d_bits || !d_packed) return HLQ_ERR_INVALID_ARGUMENT;
    if ((uintptr_t)d_bits & 7) return HLQ_ERR_ALIGNMENT;
    pack_bits_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(d_bits, d_packed, total);
    count_launch();
    return note_cuda(cudaGetLastError());
}

int hlq_unpack_bits_device(const uint8_t *d_packed, uint8_t *d_bits, int q, int64_t n, int64_t k,
                           void *stream) {
    if (q < 0 || n < 0 || k < 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (k % 8) return HLQ_ERR_SHAPE;
    const int64_t total = (int64_t)q * n * (k / 8);
    if (total == 0) return HLQ_OK;
    if (!d_bits || !d_packed) return HLQ_ERR_INVALID_ARGUMENT;
    if ((uintptr_t)d_bits & 7) return HLQ_ERR_ALIGNMENT;
    unpack_bits_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(d_packed, d_bits, total);
    count_launch();
    return note_cuda(cudaGetLastError());
}

int hlq_repack_device(const uint8_t *d_w_quant, const uint16_t *d_w_scale, const uint16_t *d_w_zero,
                      int n, int k, int g, int q, uint8_t *d_planes, uint16_t *d_meta, void *stream) {
    if (!d_w_quant || !d_w_scale || !d_w_zero || !d_planes || !d_meta) return HLQ_ERR_INVALID_ARGUMENT;
    if (n <= 0 || k <= 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (q < 1 || q > 4 || !stream_supported(g) || k % g || k % 8) return HLQ_ERR_SHAPE;
    const StreamDims d = stream_dims(n, k, g, q);
    const int64_t words = (int64_t)d.slices * d.octs * d.q * 32;
    repack_planes_kernel<<<grid_for(words, 256), 256, 0, (cudaStream_t)stream>>>(d_w_quant, d_planes, d);
    repack_meta_kernel<<<grid_for(stream_meta_elems(d), 256), 256, 0, (cudaStream_t)stream>>>(
        d_w_scale, d_w_zero, d_meta, d);
    count_launch(2);
    return note_cuda(cudaGetLastError());
}

int hlq_unrepack_device(const uint8_t *d_planes, const uint16_t *d_meta, int n, int k, int g, int q,
                        uint8_t *d_w_quant, uint16_t *d_w_scale, uint16_t *d_w_zero, void *stream) {
    if (!d_w_quant || !d_w_scale || !d_w_zero || !d_planes || !d_meta) return HLQ_ERR_INVALID_ARGUMENT;
    if (n <= 0 || k <= 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (q < 1 || q > 4 || !stream_supported(g) || k % g || k % 8) return HLQ_ERR_SHAPE;
    const StreamDims d = stream_dims(n, k, g, q);
    unrepack_planes_kernel<<<grid_for((int64_t)q * n * (k / 8), 256), 256, 0, (cudaStream_t)stream>>>(
        d_planes, d_w_quant, d);
    unrepack_meta_kernel<<<grid_for((int64_t)(q + 1) * n * (k / g), 256), 256, 0, (cudaStream_t)stream>>>(
        d_meta, d_w_scale, d_w_zero, d);
    count_launch(2);
    return note_cuda(cudaGetLastError());
}

}  // extern "C"
