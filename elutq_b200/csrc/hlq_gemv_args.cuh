// Launch arguments of the persistent GEMV kernels over the streaming layout and the walk of a
// CTA's share of a launch, shared by the LUT GEMV (hlq_gemv.cu) and the small-batch kernel
// (hlq_batch.cu); plus the launchers' host helpers.
#pragma once
#include <atomic>
#include <mutex>

#include "hlq_internal.h"

namespace hlq {

// One linear of a launch.
struct Job {
    const uint8_t *planes;
    const uint16_t *meta;
    const uint8_t *codes; // optional second copy of the planes as 4-bit code words (hlq_batch.cu), or nullptr
    const uint8_t *rcodes;   // optional: the codes once more with a row per lane, and the scales and zeros
    const uint16_t *rmeta;   // in that order (hlq_batch_tmem.cu), or nullptr
    const uint16_t *bias;
    float *acc;           // [m][np] fp32 accumulators, zero between launches
    unsigned *counters;   // [m][blocks]
    const void *x;        // [m][k]
    void *y;              // [m][n]
    int n, k, np, slices, duos, blocks;
    int x_dtype, y_dtype;
    long long unit_begin; // first (slice, duo) unit of this job in the launch
    long long unit_begin_chunked;   // the same when the launch walks the job in chunks (GemvArgs::chunk_duos)
    // Optional transform of the input while the tables are built (one row of x per pass):
    //   HLQ_INPUT_GATED_SILU:  x_eff = fp16(x2 * x / (1 + exp(-x)))
    //   HLQ_INPUT_ADD_RMSNORM: t = x + x2 (x2 may be null), res_out = fp16(t) (may be null),
    //                          x_eff = fp16(fp16(t) * gamma / sqrt(mean(t^2) + eps))
    int xop;
    float eps;
    const void *x2;          // [m][k] fp16
    const uint16_t *gamma;   // [k] fp16
    uint16_t *res_out;       // [m][k] fp16, distinct from x and x2
};

struct GemvArgs {
    const TpDev *tp;      // nullptr: no fused all-reduce
    const Job *jobs;      // njobs descriptors in global memory, or nullptr
    int njobs;            // 0: use `single`
    long long total_units;
    long long total_units_chunked;   // host only: the launch's units under the small-batch kernel's chunked walk
    int *status;
    uint32_t dyn_smem;
    int seg_cost;         // units charged per (job, slice) when the work is split over the CTAs
    int row_base;         // first row of x this launch serves (grid.y passes of R rows follow)
    int y_is_f32;         // host only: fp32 outputs keep one row per pass (fp32 table entries)
    int one_row_passes;   // host only: a job has an input transform (one row of x per pass)
    int spin_limit;       // polls after which a bounded wait gives up
    int batch_rows;       // small-batch kernel: rows of x of the launch (all served by one pass)
    int use_codes;        // small-batch kernel: every job of the launch has code words
    int use_rcodes;       // ... and row codes (then every job's duos are a multiple of 8)
    int unit_align;       // 0 or 1: a CTA's share starts anywhere; 8: on a multiple of 8 units
    int chunk_duos;       // 0: a job's units run slice by slice over all its duos; else chunk by chunk of
                          // this many duos, all slices of a chunk before the next chunk (then total_units
                          // and the jobs' unit_begin_chunked count seg_cost per (slice, chunk))
    Job single;
};

// Descriptor of one segment, written by the control warp into shared memory.
struct Seg {
    const uint8_t *planes;  // first cell of the segment
    const uint8_t *codes;   // first code words of the segment (jobs that have them), else nullptr
    const uint8_t *rcodes;  // row codes and their scales of the segment's first tile of 128 rows, else nullptr
    const uint16_t *rmeta;
    const uint16_t *meta;   // first meta entry of the segment
    const uint16_t *bias;
    float *acc;             // accumulator row base of mrow
    unsigned *counters;     // counters of mrow
    void *y;
    long long y_base;       // element offset of mrow in y
    int n, np, slices, k;
    int duo_a, duo_b;
    int x_dtype, y_dtype;
    int mrow, blocks;
    int live;
    int slice;              // slice index of the segment
    const Job *jb;          // the job (for its input transform)
};

// ---- control warp: walks the CTA's unit range and emits segment descriptors ---------------
// The launch's work is split over the CTAs in units of one duo, plus kSegCost units per
// (job, slice) for what a segment costs beside its duos (the 64 KB of tables, the barriers,
// the restart of the load ring): CTAs that get many short slices would otherwise finish last.
// Only launches of several jobs need it (a single job's slices are all alike); there
// GemvArgs::seg_cost = kSegCost, else 0.
constexpr int kSegCost = 40;
__host__ __device__ static inline long long launch_units(int slices, int duos, int seg_cost) {
    return (long long)slices * (duos + seg_cost);
}
// Chunked walk (the small-batch kernel): the blocks of a chunk complete when the chunk's last slice
// is done, so the completion work is spread over the CTAs instead of falling to whoever holds a
// job's last slice.  Its segments cost little beside their duos.
constexpr int kChunkDuos = 128;
constexpr int kCodeDuoBytes = 4096;     // code words of one duo: 16 rows x 512 channels x 4 bits
constexpr int kRowCodeTileBytes = 32768; // row codes of one tile: 128 rows x 512 channels x 4 bits, [quarter][chunk][row][16]
constexpr int kRowMetaTileBytes = 4096;  // their scales and zeros: [quarter][row][4] fp16
constexpr int kChunkSegCost = 8;     // a multiple of 8, so that cuts on multiples of 8 units fall on tiles of 8 duos
__host__ __device__ static inline long long launch_units_chunked(int slices, int duos, int chunk, int seg_cost) {
    const int chunks = (duos + chunk - 1) / chunk;
    return (long long)slices * duos + (long long)slices * chunks * seg_cost;
}

struct Walker {
    const GemvArgs *a;
    long long u, u_end;
    int jidx;
    Job jb;
    int mrow;
};

__device__ __forceinline__ long long walker_job_begin(const GemvArgs &a, const Job &jb) {
    return a.chunk_duos ? jb.unit_begin_chunked : jb.unit_begin;
}
__device__ __forceinline__ long long walker_job_units(const GemvArgs &a, const Job &jb) {
    return a.chunk_duos ? launch_units_chunked(jb.slices, jb.duos, a.chunk_duos, a.seg_cost)
                        : launch_units(jb.slices, jb.duos, a.seg_cost);
}

__device__ __forceinline__ void walker_init(Walker &w, const GemvArgs &a, int mrow) {
    w.a = &a;
    const long long al = a.unit_align > 1 ? a.unit_align : 1;
    w.u = a.total_units / al * blockIdx.x / gridDim.x * al;
    w.u_end = blockIdx.x + 1 == gridDim.x ? a.total_units : a.total_units / al * (blockIdx.x + 1) / gridDim.x * al;
    w.mrow = mrow;
    w.jidx = 0;
    if (a.njobs == 0) {
        w.jb = a.single;
    } else {
        // binary search for the job that holds unit u
        int lo = 0, hi = a.njobs - 1;
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (walker_job_begin(a, a.jobs[mid]) <= w.u) lo = mid; else hi = mid - 1;
        }
        w.jidx = lo;
        w.jb = a.jobs[lo];
    }
}

// Fills `sg` with the next segment and returns the activation slice to copy (or nullptr).
template <int Q, int GPW>
__device__ __forceinline__ const uint16_t *walker_next(Walker &w, Seg &sg, int &valid) {
    sg.live = 0;
    valid = 0;
    if (w.u >= w.u_end) return nullptr;
    const GemvArgs &a = *w.a;
    const int seg_cost = a.seg_cost;
    while (w.u >= walker_job_begin(a, w.jb) + walker_job_units(a, w.jb) && w.jidx + 1 < a.njobs) {
        ++w.jidx;
        w.jb = a.jobs[w.jidx];
    }
    const Job &jb = w.jb;
    long long local = w.u - walker_job_begin(a, jb);
    // the chunk of duos the unit lies in (one chunk = the whole job unless the walk is chunked)
    int chunk_first = 0, chunk_len = jb.duos;
    if (a.chunk_duos && jb.duos > a.chunk_duos) {
        const int chunks = (jb.duos + a.chunk_duos - 1) / a.chunk_duos;
        const long long full = (long long)jb.slices * (a.chunk_duos + seg_cost);
        long long ci = local / full;
        if (ci > chunks - 1) ci = chunks - 1;
        local -= ci * full;
        chunk_first = (int)ci * a.chunk_duos;
        chunk_len = min(a.chunk_duos, jb.duos - chunk_first);
    }
    const int per = chunk_len + seg_cost;
    const int s = (int)(local / per);
    int off = (int)(local % per);
    if (off < seg_cost) {
        // the range starts in the segment's set-up share: it owns the segment's first duos if it
        // reaches them, and nothing of this segment otherwise
        if (w.u + (seg_cost - off) >= w.u_end) {
            w.u = w.u_end;
            return nullptr;
        }
        w.u += seg_cost - off;
        off = seg_cost;
    }
    const int da = off - seg_cost;
    const long long left = w.u_end - w.u;
    const int db = (int)((long long)(chunk_len - da) < left ? chunk_len : da + left);
    const long long cell = (long long)s * jb.duos + chunk_first + da;           // in duos
    sg.planes = jb.planes + cell * (2 * Q * kCellBytes);
    sg.codes = jb.codes ? jb.codes + cell * kCodeDuoBytes : nullptr;
    sg.rcodes = nullptr;
    sg.rmeta = nullptr;
    if (jb.rcodes) {
        const long long tile = (long long)s * (jb.duos / 8) + (chunk_first + da) / 8;     // tiles of 8 duos
        sg.rcodes = jb.rcodes + tile * kRowCodeTileBytes;
        sg.rmeta = jb.rmeta + tile * (kRowMetaTileBytes / 2);
    }
    sg.meta = jb.meta + cell * ((Q + 1) * 32 * 2 * GPW);
    sg.bias = jb.bias;
    sg.acc = jb.acc + (long long)w.mrow * jb.np;
    sg.counters = jb.counters + (long long)w.mrow * jb.blocks;
    sg.y = jb.y;
    sg.y_base = (long long)w.mrow * jb.n;
    sg.n = jb.n; sg.np = jb.np; sg.slices = jb.slices; sg.k = jb.k;
    sg.duo_a = chunk_first + da; sg.duo_b = chunk_first + db;
    sg.x_dtype = jb.x_dtype; sg.y_dtype = jb.y_dtype;
    sg.mrow = w.mrow; sg.blocks = jb.blocks;
    sg.live = 1;
    sg.slice = s;
    sg.jb = a.njobs == 0 ? &a.single : &a.jobs[w.jidx];
    valid = min(kSliceK, jb.k - s * kSliceK);
    w.u += db - da;
    return (const uint16_t *)jb.x + (long long)w.mrow * jb.k + (long long)s * kSliceK;
}

// The small-batch kernel (hlq_batch.cu): whether it takes (q, m), and its launch over the jobs of `a`.
bool batch_mma_supported(int q, int m);
int launch_batch_mma(int q, int gpw, const GemvArgs &a, int ctas, int m, cudaStream_t stream);
// The same launch with the weight operand in tensor memory (hlq_batch_tmem.cu; needs a.use_rcodes).
int launch_batch_tmem(int q, int gpw, const GemvArgs &a, int ctas, int m, cudaStream_t stream);
// Row codes of a weight (g = 128, 2 or 3 bits, rows a multiple of 128) from its planes and meta.
int launch_build_row_codes(int q, const uint8_t *planes, const uint16_t *meta, uint8_t *rcodes, uint16_t *rmeta,
                           const StreamDims &d, cudaStream_t stream);
// The same launch on the tcgen05 tensor cores (hlq_batch_umma.cu).
int launch_batch_umma(int q, int gpw, const GemvArgs &a, int ctas, int m, cudaStream_t stream);
// Which of the two serves small batches: 0 = the default, 1 = mma.sync, 2 = tcgen05 (hlq_select_batch_kernel).
extern std::atomic<int> g_batch_kernel;
// The code words of a weight in the streaming layout (hlq_weight_build_batch_codes): device buffer of
// slices * duos * kCodeDuoBytes bytes from its planes.
int launch_build_codes(int q, const uint8_t *planes, uint8_t *codes, int slices, int duos, cudaStream_t stream);

// ---- host helpers of the launchers ----------------------------------------------------------
struct DeviceInfo {
    int sms = 0;
    int max_dyn_smem = 0;
    std::atomic<bool> ok{false};
};
extern std::mutex g_first_use;     // serializes the per-device lookups done on first use
// The device's SM count and shared-memory limit, looked up once; HLQ_ERR_NO_DEVICE unless sm_100.
int device_info(int device, DeviceInfo **out);

// Launch with programmatic stream serialization: the kernel may start while its predecessor
// drains and orders itself with griddepcontrol.wait.
template <typename KernelT, typename ArgsT>
static int launch_pdl(KernelT kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      const ArgsT &args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    HLQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, args));
    count_launch();
    return HLQ_OK;
}

}  // namespace hlq
