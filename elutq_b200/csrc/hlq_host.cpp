// Host-side parts of the C ABI: bit-plane packing, the streaming re-layout on the CPU,
// and status strings.  No CUDA calls in this file.
#include <cstring>

#include "../../include/hlq_b200.h"
#include "hlq_layout.h"

using namespace hlq;

extern "C" {

int hlq_abi_version(void) { return 1; }

const char *hlq_last_error_string(int status) {
    switch (status) {
        case HLQ_OK: return "ok";
        case HLQ_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, bad enum or negative size)";
        case HLQ_ERR_SHAPE: return "unsupported shape (need k % g == 0, k % 8 == 0, g % 8 == 0, 1 <= bits <= 4, valid shard split)";
        case HLQ_ERR_WORKSPACE: return "workspace missing or smaller than hlq_workspace_bytes()";
        case HLQ_ERR_CUDA: return "a CUDA runtime call failed (see hlq_last_cuda_error())";
        case HLQ_ERR_NO_DEVICE: return "no usable CUDA device (an sm_100 GPU is required)";
        case HLQ_ERR_UNSUPPORTED: return "combination not supported";
        case HLQ_ERR_ALIGNMENT: return "pointer is not aligned as documented";
        case HLQ_ERR_KERNEL: return "a kernel reported a failure through its status word";
        default: return "unknown status";
    }
}

// GPTQ/HLQ.py:239-251: packed[p, n, i] = OR_j bits[p, n, 8 i + j] << j.
int hlq_pack_bits(const uint8_t *bits, uint8_t *packed, int q, int64_t n, int64_t k) {
    if (!bits || !packed) return (q == 0 || n == 0 || k == 0) ? HLQ_OK : HLQ_ERR_INVALID_ARGUMENT;
    if (q < 0 || n < 0 || k < 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (k % 8) return HLQ_ERR_SHAPE;
    const int64_t total = (int64_t)q * n * (k / 8);
    for (int64_t i = 0; i < total; ++i) {
        const uint8_t *src = bits + i * 8;
        unsigned v = 0;
        for (int j = 0; j < 8; ++j) {
            if (src[j] > 1) return HLQ_ERR_INVALID_ARGUMENT;
            v |= (unsigned)src[j] << j;
        }
        packed[i] = (uint8_t)v;
    }
    return HLQ_OK;
}

int hlq_unpack_bits(const uint8_t *packed, uint8_t *bits, int q, int64_t n, int64_t k) {
    if (!bits || !packed) return (q == 0 || n == 0 || k == 0) ? HLQ_OK : HLQ_ERR_INVALID_ARGUMENT;
    if (q < 0 || n < 0 || k < 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (k % 8) return HLQ_ERR_SHAPE;
    const int64_t total = (int64_t)q * n * (k / 8);
    for (int64_t i = 0; i < total; ++i) {
        unsigned v = packed[i];
        for (int j = 0; j < 8; ++j) bits[i * 8 + j] = (uint8_t)((v >> j) & 1u);
    }
    return HLQ_OK;
}

static int check_stream_shape(int n, int k, int g, int q) {
    if (n <= 0 || k <= 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (q < 1 || q > 4 || !stream_supported(g) || k % g || k % 8) return HLQ_ERR_SHAPE;
    return HLQ_OK;
}

int hlq_stream_sizes(int n, int k, int g, int q, int64_t *planes_bytes, int64_t *meta_bytes) {
    int rc = check_stream_shape(n, k, g, q);
    if (rc) return rc;
    StreamDims d = stream_dims(n, k, g, q);
    if (planes_bytes) *planes_bytes = stream_planes_bytes(d);
    if (meta_bytes) *meta_bytes = stream_meta_elems(d) * 2;
    return HLQ_OK;
}

int hlq_repack_host(const uint8_t *w_quant, const uint16_t *w_scale, const uint16_t *w_zero,
                    int n, int k, int g, int q, uint8_t *planes, uint16_t *meta) {
    if (!w_quant || !w_scale || !w_zero || !planes || !meta) return HLQ_ERR_INVALID_ARGUMENT;
    int rc = check_stream_shape(n, k, g, q);
    if (rc) return rc;
    const StreamDims d = stream_dims(n, k, g, q);
    const int64_t kb = k / 8, ng = k / g;
    for (int s = 0; s < d.slices; ++s)
        for (int oct = 0; oct < d.octs; ++oct)
            for (int lane = 0; lane < 32; ++lane) {
                const int r = lane >> 2, j = lane & 3;
                const int64_t row = (int64_t)oct * kOctRows + r;
                const int64_t byte0 = (int64_t)s * (kSliceK / 8) + 16 * j;
                for (int p = 0; p < q; ++p)
                    for (int i = 0; i < 16; ++i) {
                        const int64_t sb = byte0 + stream_src_byte(i, r);
                        uint8_t v = 0;
                        if (row < n && sb < kb) v = w_quant[((int64_t)p * n + row) * kb + sb];
                        planes[stream_plane_offset(d, s, oct, p, lane, i)] = v;
                    }
                for (int pp = 0; pp <= q; ++pp)
                    for (int u = 0; u < d.gpw; ++u) {
                        const int64_t grp = ((int64_t)s * kSliceK + 128 * j) / g + stream_src_group(d, u, r);
                        uint16_t v = 0;
                        if (row < n && grp < ng)
                            v = pp < q ? w_scale[((int64_t)pp * n + row) * ng + grp]
                                       : w_zero[row * ng + grp];
                        meta[stream_meta_offset(d, s, oct, pp, lane, u)] = v;
                    }
            }
    return HLQ_OK;
}

int hlq_unrepack_host(const uint8_t *planes, const uint16_t *meta, int n, int k, int g, int q,
                      uint8_t *w_quant, uint16_t *w_scale, uint16_t *w_zero) {
    if (!w_quant || !w_scale || !w_zero || !planes || !meta) return HLQ_ERR_INVALID_ARGUMENT;
    int rc = check_stream_shape(n, k, g, q);
    if (rc) return rc;
    const StreamDims d = stream_dims(n, k, g, q);
    const int64_t kb = k / 8, ng = k / g;
    for (int64_t row = 0; row < n; ++row) {
        const int oct = (int)(row / kOctRows), r = (int)(row % kOctRows);
        for (int64_t sb = 0; sb < kb; ++sb) {
            const int s = (int)(sb / (kSliceK / 8));
            const int rem = (int)(sb % (kSliceK / 8));
            const int j = rem / 16, b = rem % 16;
            const int lane = r * 4 + j;
            for (int p = 0; p < q; ++p)
                w_quant[((int64_t)p * n + row) * kb + sb] =
                    planes[stream_plane_offset(d, s, oct, p, lane, stream_pos_of_src(b, r))];
        }
        for (int64_t grp = 0; grp < ng; ++grp) {
            const int64_t ch = grp * g;
            const int s = (int)(ch / kSliceK);
            const int j = (int)((ch % kSliceK) / 128);
            const int su = (int)((ch % 128) / g);
            const int u = su ^ (r >> d.gshift);  // XOR is its own inverse
            const int lane = r * 4 + j;
            for (int pp = 0; pp <= q; ++pp) {
                const uint16_t v = meta[stream_meta_offset(d, s, oct, pp, lane, u)];
                if (pp < q) w_scale[((int64_t)pp * n + row) * ng + grp] = v;
                else w_zero[row * ng + grp] = v;
            }
        }
    }
    return HLQ_OK;
}

}  // extern "C"
