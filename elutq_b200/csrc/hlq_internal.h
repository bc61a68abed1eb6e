// Internal declarations shared by the translation units of libhlq_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/hlq_b200.h"
#include "hlq_layout.h"

struct hlq_weight {
    int device = 0;
    int n = 0, k = 0, g = 0, q = 0;  // this shard
    int n_full = 0, k_full = 0;
    int n0 = 0, k0 = 0;              // offsets of this shard in the full weight
    int tp_rank = 0, tp_size = 1, shard_mode = 0;
    int layout = HLQ_LAYOUT_STREAM;
    // HLQ_LAYOUT_STREAM: planes = streaming cells, meta = streaming scales/zeros.
    // HLQ_LAYOUT_EXPORT: planes = uint8 [q][n][k/8]; meta = fp16 scales [q][n][k/g]
    //                    followed by fp16 zeros [n][k/g].
    uint8_t *d_planes = nullptr;
    uint16_t *d_meta = nullptr;
    uint16_t *d_bias = nullptr;
    int64_t planes_bytes = 0, meta_bytes = 0;
    // optional (streaming layout, 2 or 3 bits): the planes once more as 4-bit code words per weight,
    // which the small-batch kernel reads instead of the planes (hlq_weight_build_batch_codes)
    uint8_t *d_codes = nullptr;
    int64_t codes_bytes = 0;
    // ... and, where the shape allows (g = 128, rows a multiple of 128), the codes with a row per lane
    // plus the scales and zeros in that order, for the kernel that keeps its weight operand in tensor memory
    uint8_t *d_rcodes = nullptr;
    uint16_t *d_rmeta = nullptr;
    int64_t rcodes_bytes = 0;
    // HLQ_LAYOUT_EXPORT only: 256 zeroed bytes whose first word is the generic kernel's status
    // word when a forward call brings no workspace (allocated with the handle, never in a
    // launch path).
    int *d_status = nullptr;
    // optional extra bit-plane of the runtime's "sparse" weights: blocks of 32 rows x one group,
    // kept in exported order (coordinates of this shard)
    int sp_pairs = 0;
    uint32_t *d_sp_mask = nullptr;   // [pairs][2]
    uint8_t *d_sp_blocks = nullptr;  // [pairs][32][g/8]
    uint16_t *d_sp_scales = nullptr; // [pairs][32]
};

namespace hlq {

constexpr int kDefaultSpinLimit = 1 << 22;   // polls of one bounded wait unless the caller sets another

// Peer-mapped buffers of a fused all-reduce (one per tensor-parallel communicator), in device
// memory.  recv[p] is rank p's receive buffer as mapped into this
// process; slot (parity, source rank, row of x, output row or block).
struct TpDev {
    unsigned long long *recv[8];   // slots of (launch number << 32 | fp32 bits): value and flag are one 64-bit word
    unsigned *seq;        // number of finished fused launches on this rank
    unsigned *done;       // blocks summed so far in the current launch
    int rank, world, max_m, np_cap;
};

}  // namespace hlq

struct hlq_tp_comm {
    int device = 0, rank = 0, world = 1, max_m = 1, np_cap = 0;
    unsigned char *local = nullptr;      // this rank's receive buffer, flags, counters (cudaMalloc)
    size_t bytes = 0, seq_off = 0;
    void *peer[8] = {};                  // every rank's buffer as mapped here
    hlq::TpDev *d_tp = nullptr;
    bool connected = false;
    bool ipc = false;                    // peer[] came from cudaIpcOpenMemHandle
    int spin_limit = hlq::kDefaultSpinLimit;
};

namespace hlq {

// Records a failing CUDA call for hlq_last_cuda_error(); returns HLQ_ERR_CUDA or HLQ_OK.
int note_cuda(cudaError_t e);
void count_launch(int n = 1);

#define HLQ_CUDA(call)                                  \
    do {                                                \
        cudaError_t e__ = (call);                       \
        if (e__ != cudaSuccess) return hlq::note_cuda(e__); \
    } while (0)

// Workspace layout: [0, 256) header (int status at 0), then counters, then accumulators.
constexpr size_t kWsHeader = 256;
constexpr int kLutMaxM = 16;  // rows of x one LUT-GEMV launch handles

struct Workspace {
    int *status;
    unsigned *counters;  // [m][blocks]
    float *partial;      // [m][np] fp32 accumulators
};
size_t workspace_bytes_for(int m, const StreamDims &d);
size_t gemm_scratch_offset(const StreamDims &d);   // byte offset of the GEMM's fp16 copy of bf16 activations
size_t gemm_acc_offset(int m, const StreamDims &d); // ... and of its fp32 sums when K is split
constexpr int kGemmSplitMaxM = 256;                // rows of x up to which the workspace holds room for them
constexpr size_t kGemmSlabBytes = 16u << 20;       // ... at most this much (up to 8 slabs)
Workspace carve_workspace(void *base, int m, const StreamDims &d);

// Kernels' launchers (defined in the .cu files).  All return an hlq_status.
int launch_lut8_gemv(const hlq_weight *w, int m, const void *x, int x_dtype, void *y, int y_dtype,
                     void *workspace, size_t workspace_bytes, cudaStream_t stream,
                     const hlq_input_op *op = nullptr);
int launch_lut4_gemv(const hlq_weight *w, int m, const void *x, int x_dtype, void *y, int y_dtype,
                     void *workspace, size_t workspace_bytes, cudaStream_t stream);
// The extra bit-plane of a weight that has one (hlq_sparse.cu): into fp32 accumulators [m][acc_stride] when
// `acc` is given, else added to y in place.  No-op for weights without the plane.
int launch_sparse_plane(const hlq_weight *w, int m, const void *x, int x_dtype, float *acc, int acc_stride, void *y,
                        int y_dtype, cudaStream_t stream);
void free_sparse(hlq_weight *w);
// Splits of the context per kv head the attention kernel uses for a cache of max_ctx positions.
int attention_splits(int head_kv, int max_ctx);
int launch_dequant_gemm(const hlq_weight *w, int m, const void *x, int x_dtype, void *y,
                        int y_dtype, void *workspace, size_t workspace_bytes,
                        cudaStream_t stream);

}  // namespace hlq
