// C ABI: weight handles, workspace and the forward dispatcher.
//
// Replaces the reference's operator layer for the quantized linear:
//   load_Parameter            C++/ops/src/arm/parameters.cpp:5-70
//   weight_tensor             C++/ops/include/arm/arm_nnstructures.h:11-37
//   arm_gemm (dispatcher)     C++/ops/src/arm/arm_gemm.cpp:871-924
#include <atomic>
#include <cstring>
#include <new>
#include <vector>

#include "hlq_gemv_args.cuh"
#include "hlq_internal.h"

namespace hlq {

static thread_local int g_last_cuda_error = 0;
static std::atomic<int64_t> g_launches{0};

int note_cuda(cudaError_t e) {
    if (e == cudaSuccess) return HLQ_OK;
    g_last_cuda_error = (int)e;
    (void)cudaGetLastError();  // clear the sticky flag of non-fatal errors
    return HLQ_ERR_CUDA;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

static int check_shape(int n, int k, int g, int q) {
    if (n <= 0 || k <= 0 || g <= 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (q < 1 || q > 4 || k % g || k % 8 || g % 8) return HLQ_ERR_SHAPE;
    return HLQ_OK;
}

struct ShardPlan {
    int n, k;          // shard sizes
    int n0, k0;        // offsets into the full weight
};

static int plan_shard(int n_full, int k_full, int g, int rank, int size, int mode, ShardPlan *out) {
    ShardPlan s{n_full, k_full, 0, 0};
    if (size < 1 || rank < 0 || rank >= size) return HLQ_ERR_INVALID_ARGUMENT;
    if (mode != HLQ_SHARD_NONE && mode != HLQ_SHARD_ROWS && mode != HLQ_SHARD_COLS)
        return HLQ_ERR_INVALID_ARGUMENT;
    if (size > 1 && mode == HLQ_SHARD_ROWS) {
        if (n_full % size) return HLQ_ERR_SHAPE;
        s.n = n_full / size;
        s.n0 = rank * s.n;
    } else if (size > 1 && mode == HLQ_SHARD_COLS) {
        // whole groups and whole 128-channel lane words per rank
        const int unit = (g > 128 && g % 128 == 0) ? g : ((128 % g == 0) ? 128 : g);
        if (k_full % size || (k_full / size) % unit) return HLQ_ERR_SHAPE;
        s.k = k_full / size;
        s.k0 = rank * s.k;
    }
    *out = s;
    return HLQ_OK;
}

// Copies a [rows x row_bytes] window of a pitched host-or-device array to the device.
static int upload_2d(void *dst, const void *src, size_t src_pitch, size_t row_bytes, size_t rows,
                     cudaStream_t stream) {
    if (rows == 0 || row_bytes == 0) return HLQ_OK;
    HLQ_CUDA(cudaMemcpy2DAsync(dst, row_bytes, src, src_pitch, row_bytes, rows, cudaMemcpyDefault,
                               stream));
    return HLQ_OK;
}

struct DeviceGuard {
    int prev = -1;
    bool set(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) return false;
        return cudaSetDevice(dev) == cudaSuccess;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

static int alloc_buffers(hlq_weight *w, bool with_bias) {
    if (w->layout == HLQ_LAYOUT_STREAM) {
        const StreamDims d = stream_dims(w->n, w->k, w->g, w->q);
        w->planes_bytes = stream_planes_bytes(d);
        w->meta_bytes = stream_meta_elems(d) * 2;
    } else {
        w->planes_bytes = (int64_t)w->q * w->n * (w->k / 8);
        w->meta_bytes = (int64_t)(w->q + 1) * w->n * (w->k / w->g) * 2;
    }
    HLQ_CUDA(cudaMalloc((void **)&w->d_planes, (size_t)w->planes_bytes));
    HLQ_CUDA(cudaMalloc((void **)&w->d_meta, (size_t)w->meta_bytes));
    if (with_bias) HLQ_CUDA(cudaMalloc((void **)&w->d_bias, (size_t)w->n * 2));
    if (w->layout == HLQ_LAYOUT_EXPORT) {
        HLQ_CUDA(cudaMalloc((void **)&w->d_status, kWsHeader));
        HLQ_CUDA(cudaMemset(w->d_status, 0, kWsHeader));
    }
    return HLQ_OK;
}

static void free_buffers(hlq_weight *w) {
    if (w->d_planes) cudaFree(w->d_planes);
    if (w->d_meta) cudaFree(w->d_meta);
    if (w->d_bias) cudaFree(w->d_bias);
    if (w->d_status) cudaFree(w->d_status);
    w->d_status = nullptr;
    if (w->d_codes) cudaFree(w->d_codes);
    w->d_codes = nullptr;
    w->codes_bytes = 0;
    if (w->d_rcodes) cudaFree(w->d_rcodes);
    if (w->d_rmeta) cudaFree(w->d_rmeta);
    w->d_rcodes = nullptr;
    w->d_rmeta = nullptr;
    w->rcodes_bytes = 0;
    free_sparse(w);
    w->d_planes = nullptr;
    w->d_meta = nullptr;
    w->d_bias = nullptr;
}

}  // namespace hlq

using namespace hlq;

extern "C" {

int hlq_last_cuda_error(void) { return g_last_cuda_error; }
int64_t hlq_kernel_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int hlq_weight_alloc(hlq_weight **out, int in_ch, int out_ch, int g, int q, int has_bias, int device,
                     unsigned flags) {
    if (!out) return HLQ_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    int rc = check_shape(out_ch, in_ch, g, q);
    if (rc) return rc;
    DeviceGuard guard;
    if (!guard.set(device)) {
        note_cuda(cudaGetLastError());
        return HLQ_ERR_NO_DEVICE;
    }
    hlq_weight *w = new (std::nothrow) hlq_weight();
    if (!w) return HLQ_ERR_INVALID_ARGUMENT;
    w->device = device;
    w->n = w->n_full = out_ch;
    w->k = w->k_full = in_ch;
    w->g = g;
    w->q = q;
    w->layout = (stream_supported(g) && !(flags & HLQ_FLAG_FORCE_EXPORT_LAYOUT)) ? HLQ_LAYOUT_STREAM
                                                                                 : HLQ_LAYOUT_EXPORT;
    rc = alloc_buffers(w, has_bias != 0);
    if (rc) {
        free_buffers(w);
        delete w;
        return rc;
    }
    *out = w;
    return HLQ_OK;
}

int hlq_weight_from_export(hlq_weight **out, const void *w_quant, const void *w_scale,
                           const void *w_zero, const void *bias, int in_ch, int out_ch, int g, int q,
                           int device, int tp_rank, int tp_size, int shard_mode, unsigned flags,
                           void *stream_) {
    if (!out) return HLQ_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (!w_quant || !w_scale || !w_zero) return HLQ_ERR_INVALID_ARGUMENT;
    int rc = check_shape(out_ch, in_ch, g, q);
    if (rc) return rc;
    ShardPlan sp;
    rc = plan_shard(out_ch, in_ch, g, tp_rank, tp_size, shard_mode, &sp);
    if (rc) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    DeviceGuard guard;
    if (!guard.set(device)) {
        note_cuda(cudaGetLastError());
        return HLQ_ERR_NO_DEVICE;
    }

    hlq_weight *w = new (std::nothrow) hlq_weight();
    if (!w) return HLQ_ERR_INVALID_ARGUMENT;
    w->device = device;
    w->n = sp.n; w->k = sp.k; w->g = g; w->q = q;
    w->n_full = out_ch; w->k_full = in_ch;
    w->n0 = sp.n0; w->k0 = sp.k0;
    w->tp_rank = tp_rank; w->tp_size = tp_size; w->shard_mode = tp_size > 1 ? shard_mode : HLQ_SHARD_NONE;
    w->layout = (stream_supported(g) && !(flags & HLQ_FLAG_FORCE_EXPORT_LAYOUT)) ? HLQ_LAYOUT_STREAM
                                                                                 : HLQ_LAYOUT_EXPORT;
    const bool keep_bias = bias && !(w->shard_mode == HLQ_SHARD_COLS && tp_rank != 0);
    rc = alloc_buffers(w, keep_bias);

    // Stage the shard in exported order on the device (directly into the handle when the
    // handle keeps the exported layout), then re-lay-out with a kernel.
    const int64_t kb_full = in_ch / 8, ng_full = in_ch / g;
    const int64_t kb = sp.k / 8, ng = sp.k / g;
    const int64_t quant_bytes = (int64_t)q * sp.n * kb;
    const int64_t scale_elems = (int64_t)q * sp.n * ng;
    const int64_t zero_elems = (int64_t)sp.n * ng;
    uint8_t *st_quant = nullptr;
    uint16_t *st_meta = nullptr;
    bool staged = false;
    if (!rc) {
        if (w->layout == HLQ_LAYOUT_EXPORT) {
            st_quant = w->d_planes;
            st_meta = w->d_meta;
        } else {
            staged = true;
            if (cudaMalloc((void **)&st_quant, (size_t)quant_bytes) != cudaSuccess ||
                cudaMalloc((void **)&st_meta, (size_t)(scale_elems + zero_elems) * 2) != cudaSuccess)
                rc = note_cuda(cudaErrorMemoryAllocation);
        }
    }
    if (!rc) {
        for (int p = 0; p < q && !rc; ++p) {
            const uint8_t *src = (const uint8_t *)w_quant + ((int64_t)p * out_ch + sp.n0) * kb_full + sp.k0 / 8;
            rc = upload_2d(st_quant + (int64_t)p * sp.n * kb, src, (size_t)kb_full, (size_t)kb,
                           (size_t)sp.n, stream);
            if (rc) break;
            const uint16_t *ss = (const uint16_t *)w_scale + ((int64_t)p * out_ch + sp.n0) * ng_full + sp.k0 / g;
            rc = upload_2d(st_meta + (int64_t)p * sp.n * ng, ss, (size_t)ng_full * 2, (size_t)ng * 2,
                           (size_t)sp.n, stream);
        }
        if (!rc) {
            const uint16_t *zs = (const uint16_t *)w_zero + (int64_t)sp.n0 * ng_full + sp.k0 / g;
            rc = upload_2d(st_meta + scale_elems, zs, (size_t)ng_full * 2, (size_t)ng * 2, (size_t)sp.n,
                           stream);
        }
        if (!rc && keep_bias)
            rc = upload_2d(w->d_bias, (const uint16_t *)bias + sp.n0, (size_t)sp.n * 2, (size_t)sp.n * 2, 1,
                           stream);
    }
    if (!rc && staged)
        rc = hlq_repack_device(st_quant, st_meta, st_meta + scale_elems, sp.n, sp.k, g, q, w->d_planes,
                               w->d_meta, stream);
    if (!rc) rc = note_cuda(cudaStreamSynchronize(stream));
    if (staged) {
        if (st_quant) cudaFree(st_quant);
        if (st_meta) cudaFree(st_meta);
    }
    if (rc) {
        free_buffers(w);
        delete w;
        return rc;
    }
    *out = w;
    return HLQ_OK;
}

int hlq_weight_to_export(const hlq_weight *w, void *h_w_quant, void *h_w_scale, void *h_w_zero,
                         void *h_bias, void *stream_) {
    if (!w || !h_w_quant || !h_w_scale || !h_w_zero) return HLQ_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = (cudaStream_t)stream_;
    DeviceGuard guard;
    if (!guard.set(w->device)) return HLQ_ERR_NO_DEVICE;
    const int64_t kb = w->k / 8, ng = w->k / w->g;
    const int64_t quant_bytes = (int64_t)w->q * w->n * kb;
    const int64_t scale_elems = (int64_t)w->q * w->n * ng;
    const int64_t zero_elems = (int64_t)w->n * ng;
    int rc = HLQ_OK;
    if (w->layout == HLQ_LAYOUT_EXPORT) {
        HLQ_CUDA(cudaMemcpyAsync(h_w_quant, w->d_planes, (size_t)quant_bytes, cudaMemcpyDeviceToHost, stream));
        HLQ_CUDA(cudaMemcpyAsync(h_w_scale, w->d_meta, (size_t)scale_elems * 2, cudaMemcpyDeviceToHost, stream));
        HLQ_CUDA(cudaMemcpyAsync(h_w_zero, w->d_meta + scale_elems, (size_t)zero_elems * 2,
                                 cudaMemcpyDeviceToHost, stream));
    } else {
        uint8_t *tq = nullptr;
        uint16_t *tm = nullptr;
        HLQ_CUDA(cudaMalloc((void **)&tq, (size_t)quant_bytes));
        if (cudaMalloc((void **)&tm, (size_t)(scale_elems + zero_elems) * 2) != cudaSuccess) {
            cudaFree(tq);
            return note_cuda(cudaErrorMemoryAllocation);
        }
        rc = hlq_unrepack_device(w->d_planes, w->d_meta, w->n, w->k, w->g, w->q, tq, tm, tm + scale_elems,
                                 stream);
        if (!rc) rc = note_cuda(cudaMemcpyAsync(h_w_quant, tq, (size_t)quant_bytes, cudaMemcpyDeviceToHost, stream));
        if (!rc) rc = note_cuda(cudaMemcpyAsync(h_w_scale, tm, (size_t)scale_elems * 2, cudaMemcpyDeviceToHost, stream));
        if (!rc) rc = note_cuda(cudaMemcpyAsync(h_w_zero, tm + scale_elems, (size_t)zero_elems * 2,
                                                cudaMemcpyDeviceToHost, stream));
        if (!rc) rc = note_cuda(cudaStreamSynchronize(stream));
        cudaFree(tq);
        cudaFree(tm);
        if (rc) return rc;
    }
    if (h_bias && w->d_bias)
        HLQ_CUDA(cudaMemcpyAsync(h_bias, w->d_bias, (size_t)w->n * 2, cudaMemcpyDeviceToHost, stream));
    HLQ_CUDA(cudaStreamSynchronize(stream));
    return HLQ_OK;
}

int hlq_weight_free(hlq_weight *w) {
    if (!w) return HLQ_OK;
    DeviceGuard guard;
    guard.set(w->device);
    free_buffers(w);
    delete w;
    return HLQ_OK;
}

int hlq_weight_get_info(const hlq_weight *w, hlq_weight_info *info) {
    if (!w || !info) return HLQ_ERR_INVALID_ARGUMENT;
    info->in_channel = w->k;
    info->out_channel = w->n;
    info->groupsize = w->g;
    info->bits = w->q;
    info->has_bias = w->d_bias != nullptr;
    info->layout = w->layout;
    info->device = w->device;
    info->tp_rank = w->tp_rank;
    info->tp_size = w->tp_size;
    info->shard_mode = w->shard_mode;
    info->full_in_channel = w->k_full;
    info->full_out_channel = w->n_full;
    info->device_bytes = w->planes_bytes + w->meta_bytes + w->codes_bytes + w->rcodes_bytes + (w->d_bias ? (int64_t)w->n * 2 : 0);
    info->algorithmic_bytes = (int64_t)w->q * w->n * (w->k / 8) + 2 * (int64_t)(w->q + 1) * w->n * (w->k / w->g);
    return HLQ_OK;
}

int hlq_weight_buffers(const hlq_weight *w, void **d_planes, int64_t *planes_bytes, void **d_meta,
                       int64_t *meta_bytes, void **d_bias) {
    if (!w) return HLQ_ERR_INVALID_ARGUMENT;
    if (d_planes) *d_planes = w->d_planes;
    if (planes_bytes) *planes_bytes = w->planes_bytes;
    if (d_meta) *d_meta = w->d_meta;
    if (meta_bytes) *meta_bytes = w->meta_bytes;
    if (d_bias) *d_bias = w->d_bias;
    return HLQ_OK;
}

int hlq_weight_build_batch_codes(hlq_weight *w, void *stream) {
    if (!w) return HLQ_ERR_INVALID_ARGUMENT;
    if (w->layout != HLQ_LAYOUT_STREAM || (w->q != 2 && w->q != 3)) return HLQ_ERR_UNSUPPORTED;
    if (w->d_codes) return HLQ_OK;
    int cur = -1;
    HLQ_CUDA(cudaGetDevice(&cur));
    if (cur != w->device) return HLQ_ERR_INVALID_ARGUMENT;
    const StreamDims d = stream_dims(w->n, w->k, w->g, w->q);
    const int64_t bytes = (int64_t)d.slices * d.duos * hlq::kCodeDuoBytes;
    uint8_t *p = nullptr;
    HLQ_CUDA(cudaMalloc((void **)&p, (size_t)bytes));
    const int rc = hlq::launch_build_codes(w->q, w->d_planes, p, d.slices, d.duos, (cudaStream_t)stream);
    if (rc) {
        cudaFree(p);
        return rc;
    }
    w->d_codes = p;
    w->codes_bytes = bytes;
    // where the shape allows, also the codes with a row per lane (hlq_batch_tmem.cu)
    if (w->g == 128 && d.np % 128 == 0) {
        const int64_t tiles = (int64_t)d.slices * (d.np / 128);
        uint8_t *rc = nullptr;
        uint16_t *rm = nullptr;
        if (cudaMalloc((void **)&rc, (size_t)(tiles * hlq::kRowCodeTileBytes)) == cudaSuccess &&
            cudaMalloc((void **)&rm, (size_t)(tiles * hlq::kRowMetaTileBytes)) == cudaSuccess &&
            hlq::launch_build_row_codes(w->q, w->d_planes, w->d_meta, rc, rm, d, (cudaStream_t)stream) == HLQ_OK) {
            w->d_rcodes = rc;
            w->d_rmeta = rm;
            w->rcodes_bytes = tiles * (hlq::kRowCodeTileBytes + hlq::kRowMetaTileBytes);
        } else {
            if (rc) cudaFree(rc);
            if (rm) cudaFree(rm);
            return hlq::note_cuda(cudaGetLastError()) ? HLQ_ERR_CUDA : HLQ_ERR_CUDA;
        }
    }
    return HLQ_OK;
}

size_t hlq_workspace_bytes(int m, int k, int n, int q, int g) {
    if (m <= 0 || k <= 0 || n <= 0 || q < 1 || q > 4) return 0;
    const int gg = stream_supported(g) ? g : 128;
    return workspace_bytes_for(m, stream_dims(n, k, gg, q));
}

int hlq_workspace_init(void *d_workspace, size_t bytes, void *stream) {
    if (bytes == 0) return HLQ_OK;
    if (!d_workspace) return HLQ_ERR_INVALID_ARGUMENT;
    HLQ_CUDA(cudaMemsetAsync(d_workspace, 0, bytes, (cudaStream_t)stream));
    return HLQ_OK;
}

int hlq_workspace_status(const void *d_workspace, void *stream, int *kernel_status) {
    if (!d_workspace || !kernel_status) return HLQ_ERR_INVALID_ARGUMENT;
    HLQ_CUDA(cudaMemcpyAsync(kernel_status, d_workspace, sizeof(int), cudaMemcpyDeviceToHost,
                             (cudaStream_t)stream));
    HLQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return *kernel_status ? HLQ_ERR_KERNEL : HLQ_OK;
}

int hlq_linear_forward_op(int m, int k, int n, const void *d_x, int x_dtype, void *d_y, int y_dtype,
                          void *d_workspace, size_t workspace_bytes, const hlq_weight *w, const hlq_input_op *op,
                          void *stream_) {
    if (!w || m < 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (k != w->k || n != w->n) return HLQ_ERR_SHAPE;
    if (m == 0) return HLQ_OK;
    if (!d_x || !d_y) return HLQ_ERR_INVALID_ARGUMENT;
    if (m > hlq::kLutMaxM) return HLQ_ERR_UNSUPPORTED;
    if (y_dtype != HLQ_F16 && y_dtype != HLQ_BF16 && y_dtype != HLQ_F32) return HLQ_ERR_UNSUPPORTED;
    if (w->sp_pairs && op && op->kind != HLQ_INPUT_PLAIN) return HLQ_ERR_UNSUPPORTED;   // the plane sees plain x
    int cur = -1;
    HLQ_CUDA(cudaGetDevice(&cur));
    if (cur != w->device) return HLQ_ERR_INVALID_ARGUMENT;
    return hlq::launch_lut8_gemv(w, m, d_x, x_dtype, d_y, y_dtype, d_workspace, workspace_bytes,
                                 (cudaStream_t)stream_, op);
}

int hlq_linear_forward_impl(int impl, int m, int k, int n, const void *d_x, int x_dtype, void *d_y,
                            int y_dtype, void *d_workspace, size_t workspace_bytes, const hlq_weight *w,
                            void *stream_) {
    if (!w || m < 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (k != w->k || n != w->n) return HLQ_ERR_SHAPE;
    if (m == 0) return HLQ_OK;
    if (!d_x || !d_y) return HLQ_ERR_INVALID_ARGUMENT;
    if (x_dtype != HLQ_F16 && x_dtype != HLQ_BF16) return HLQ_ERR_UNSUPPORTED;
    if (y_dtype != HLQ_F16 && y_dtype != HLQ_BF16 && y_dtype != HLQ_F32) return HLQ_ERR_UNSUPPORTED;
    cudaStream_t stream = (cudaStream_t)stream_;
    int cur = -1;
    HLQ_CUDA(cudaGetDevice(&cur));
    if (cur != w->device) return HLQ_ERR_INVALID_ARGUMENT;
    if (impl == 0) {
        // exported layout -> generic kernel; up to 16 rows -> the LUT GEMV and the small-batch
        // kernel; more -> dequantize + tensor-core GEMM (measured on a Llama-3-8B layer at w3g128:
        // 32 rows as two launches of 16 take 289 us, the GEMM 140 us for any m up to 128).
        if (w->layout == HLQ_LAYOUT_EXPORT) impl = 2;
        else impl = m <= kLutMaxM ? 1 : 3;
    }
    int rc;
    switch (impl) {
        // the LUT GEMV takes the extra bit-plane into its accumulators before it runs
        case 1: return launch_lut8_gemv(w, m, d_x, x_dtype, d_y, y_dtype, d_workspace, workspace_bytes, stream);
        case 2: rc = launch_lut4_gemv(w, m, d_x, x_dtype, d_y, y_dtype, d_workspace, workspace_bytes, stream); break;
        case 3: rc = launch_dequant_gemm(w, m, d_x, x_dtype, d_y, y_dtype, d_workspace, workspace_bytes, stream); break;
        default: return HLQ_ERR_INVALID_ARGUMENT;
    }
    // the other kernels: the extra bit-plane is added to y afterwards
    if (!rc && w->sp_pairs) rc = launch_sparse_plane(w, m, d_x, x_dtype, nullptr, 0, d_y, y_dtype, stream);
    return rc;
}

int hlq_linear_forward(int m, int k, int n, const void *d_x, int x_dtype, void *d_y, int y_dtype,
                       void *d_workspace, size_t workspace_bytes, const hlq_weight *w, void *stream) {
    return hlq_linear_forward_impl(0, m, k, n, d_x, x_dtype, d_y, y_dtype, d_workspace, workspace_bytes, w,
                                   stream);
}

}  // extern "C"
