/*
 * hlq_b200 -- C ABI of the B200 (sm_100a) implementation of ELUTQ's quantized-linear path.
 *
 * HLQ (Hierarchical Linear Quantization): each group of g input channels of one output
 * row is stored as q binary bit-planes b_i in {0,1}, one fp16 scale alpha_i per plane and
 * one fp16 offset z, so that  w = sum_i alpha_i * b_i + z.
 *
 * The entry points mirror the reference's operator interface for this path; each
 * declaration names the reference interface it replaces (paths relative to the ELUTQ
 * project root).  The reference has no FFI layer: its interface is a direct C++ call
 * (arm_gemm + weight_tensor + load_Parameter) and the on-disk export format.
 *
 * Conventions
 *  - every function returns an hlq_status (0 = HLQ_OK); nothing exits or throws;
 *  - pointers named d_* are device pointers, h_* host pointers; plain names accept either
 *    where the comment says so;
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream);
 *    device work is enqueued on it and the call returns without synchronizing unless the
 *    comment says otherwise;
 *  - tensors are row-major; activations x are [m, k], outputs y are [m, n].
 */
#ifndef HLQ_B200_H
#define HLQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum hlq_status {
    HLQ_OK = 0,
    HLQ_ERR_INVALID_ARGUMENT = 1, /* null pointer, bad enum value, negative size            */
    HLQ_ERR_SHAPE = 2,            /* k % g, k % 8, g % 8, bits outside 1..4, bad shard split */
    HLQ_ERR_WORKSPACE = 3,        /* workspace missing or smaller than hlq_workspace_bytes   */
    HLQ_ERR_CUDA = 4,             /* a CUDA runtime call failed (see hlq_last_cuda_error)    */
    HLQ_ERR_NO_DEVICE = 5,        /* no CUDA device / wrong architecture (needs sm_100)      */
    HLQ_ERR_UNSUPPORTED = 6,      /* combination not implemented (e.g. dtype)                */
    HLQ_ERR_ALIGNMENT = 7,        /* pointer not aligned as documented                       */
    HLQ_ERR_KERNEL = 8            /* a kernel reported a failure through its status word     */
} hlq_status;

typedef enum hlq_dtype { HLQ_F16 = 0, HLQ_BF16 = 1, HLQ_F32 = 2 } hlq_dtype;

/* How a weight is cut for tensor parallelism when it is loaded. */
typedef enum hlq_shard_mode {
    HLQ_SHARD_NONE = 0,
    HLQ_SHARD_ROWS = 1, /* column-parallel: output rows n are split; no collective needed    */
    HLQ_SHARD_COLS = 2  /* row-parallel: input channels k are split (whole groups, multiples */
                        /* of 128 channels); outputs of the ranks must be summed             */
} hlq_shard_mode;

/* Device-side storage of a loaded weight. */
typedef enum hlq_layout {
    HLQ_LAYOUT_STREAM = 0, /* slice/oct streaming layout of the LUT GEMV (g in 32, 64, 128) */
    HLQ_LAYOUT_EXPORT = 1  /* the exported arrays kept as they are (any g % 8 == 0)          */
} hlq_layout;

/* Flags of hlq_weight_from_export. */
#define HLQ_FLAG_FORCE_EXPORT_LAYOUT 1u /* keep the exported arrays; use the generic kernel */

/* Opaque handle that owns the device buffers of one quantized linear.
 * Replaces: class weight_tensor, C++/ops/include/arm/arm_nnstructures.h:11-37. */
typedef struct hlq_weight hlq_weight;

typedef struct hlq_weight_info {
    int in_channel;      /* k of this shard                       */
    int out_channel;     /* n of this shard                       */
    int groupsize;       /* g                                     */
    int bits;            /* q                                     */
    int has_bias;
    int layout;          /* hlq_layout                            */
    int device;
    int tp_rank, tp_size, shard_mode;
    int full_in_channel, full_out_channel; /* before sharding     */
    int64_t device_bytes;    /* bytes this handle holds on the device              */
    int64_t algorithmic_bytes; /* q*n*k/8 + 2*(q+1)*n*k/g: planes + fp16 scales + fp16 zeros */
} hlq_weight_info;

/* ---- quantizer step ----------------------------------------------------------------- */

/* Assignment step of the reference's quantizer on the device: for every element of
 * w [blocks][g] (fp32) the nearest of the 2^q values sum_j scales[b][j] * c_j to w - zeros[b],
 * first minimum on ties; out is uint8 [blocks][g][q] of 0/1 (column j pairs with scale j).
 * Replaces: quantize_with_scales, GPTQ/quant.py:154-174. */
int hlq_quantize_with_scales_device(const float *d_w, const float *d_scales, const float *d_zeros,
                                    uint8_t *d_out, int64_t blocks, int g, int q, void *stream);

/* The fit that precedes the assignment: for every block of g weights (fp32 [blocks][g]) the q plane scales
 * and the offset that minimize the squared error, found by alternating `iters` times (the reference uses
 * 10) between assigning every weight to the nearest of the 2^q values and solving the (q+1) x (q+1) normal
 * equations for scales and offset (pseudo-inverse: a plane that no weight uses gets scale 0).  Start: plane j
 * = range / (2^q - 1) * 2^j, offset = minimum.  scales fp32 [blocks][q], zeros fp32 [blocks]; g <= 1024.
 * hlq_fit_alternating_device + hlq_quantize_with_scales_device + hlq_pack_bits_device produce, on the device,
 * what the reference's pseudo_quantize_tensor(use_alternating_optimization=True) and its exporter produce.
 * Replaces: find_optimal_params_alternating, GPTQ/quant.py:118-153, with optimize_s_batch_with_constant,
 * GPTQ/quant.py:104-116. */
int hlq_fit_alternating_device(const float *d_w, float *d_scales, float *d_zeros, int64_t blocks, int g, int q,
                               int iters, void *stream);

/* ---- bit-plane packing -------------------------------------------------------------- */

/* bits: uint8 [q][n][k] of 0/1  ->  packed: uint8 [q][n][k/8]; channel 8i+j goes to bit j
 * of byte i (bit 0 = lowest channel).  Host buffers, runs on the calling thread.
 * Replaces: HLQ.Pack_T_MAC_Weight, GPTQ/HLQ.py:239-251. */
int hlq_pack_bits(const uint8_t *h_bits, uint8_t *h_packed, int q, int64_t n, int64_t k);
/* Inverse of hlq_pack_bits (the reference has no unpacker; this is the exact inverse of
 * GPTQ/HLQ.py:239-251). */
int hlq_unpack_bits(const uint8_t *h_packed, uint8_t *h_bits, int q, int64_t n, int64_t k);
/* The same two operations on device buffers, as CUDA kernels on `stream`. */
int hlq_pack_bits_device(const uint8_t *d_bits, uint8_t *d_packed, int q, int64_t n, int64_t k,
                         void *stream);
int hlq_unpack_bits_device(const uint8_t *d_packed, uint8_t *d_bits, int q, int64_t n,
                           int64_t k, void *stream);

/* ---- streaming layout (load-time re-layout) ----------------------------------------- */

/* Sizes, in bytes, of the streaming-layout buffers of an [n, k] weight.
 * Replaces the size arithmetic of load_Parameter, C++/ops/src/arm/parameters.cpp:34-50. */
int hlq_stream_sizes(int n, int k, int groupsize, int bits, int64_t *planes_bytes,
                     int64_t *meta_bytes);
/* Exported arrays -> streaming layout, on the host (reference implementation of the
 * layout, also usable to prepare buffers off-line).  w_quant uint8 [q][n][k/8], w_scale
 * fp16 [q][n][k/g], w_zero fp16 [n][k/g].
 * Replaces: t_mac_g4_rearrange_weight_normal_impl, C++/ops/src/arm/arm_t_mac_kernal.cpp:472-552. */
int hlq_repack_host(const uint8_t *h_w_quant, const uint16_t *h_w_scale,
                    const uint16_t *h_w_zero, int n, int k, int groupsize, int bits,
                    uint8_t *h_planes, uint16_t *h_meta);
/* Exact inverse of hlq_repack_host. */
int hlq_unrepack_host(const uint8_t *h_planes, const uint16_t *h_meta, int n, int k,
                      int groupsize, int bits, uint8_t *h_w_quant, uint16_t *h_w_scale,
                      uint16_t *h_w_zero);
/* The same as CUDA kernels on device buffers. */
int hlq_repack_device(const uint8_t *d_w_quant, const uint16_t *d_w_scale,
                      const uint16_t *d_w_zero, int n, int k, int groupsize, int bits,
                      uint8_t *d_planes, uint16_t *d_meta, void *stream);
int hlq_unrepack_device(const uint8_t *d_planes, const uint16_t *d_meta, int n, int k,
                        int groupsize, int bits, uint8_t *d_w_quant, uint16_t *d_w_scale,
                        uint16_t *d_w_zero, void *stream);

/* ---- weights ------------------------------------------------------------------------ */

/* Build a device-resident weight from the exported arrays of ONE linear:
 *   w_quant uint8 [bits][out_ch][in_ch/8], w_scale fp16 [bits][out_ch][in_ch/g],
 *   w_zero fp16 [out_ch][in_ch/g], bias fp16 [out_ch] or NULL.
 * The four pointers may be host or device pointers (detected).  in_ch/out_ch are the FULL
 * sizes; with tp_size > 1 only the shard of tp_rank is uploaded and kept (shard_mode
 * says how; with HLQ_SHARD_COLS the bias is kept by rank 0 only).  The call selects
 * `device`, synchronizes `stream` before returning, and the handle owns its buffers.
 * Replaces: load_Parameter(PARAM_TYPE_LINEAR), C++/ops/src/arm/parameters.cpp:5-70, and
 * the re-layout it calls (arm_t_mac_kernal.cpp:652-674). */
int hlq_weight_from_export(hlq_weight **out, const void *w_quant, const void *w_scale,
                           const void *w_zero, const void *bias_or_null, int in_ch, int out_ch,
                           int groupsize, int bits, int device, int tp_rank, int tp_size,
                           int shard_mode, unsigned flags, void *stream);
/* Write this handle's shard back as exported arrays into HOST buffers sized for the shard
 * (bias may be NULL).  Synchronizes.  Bit-exact inverse of hlq_weight_from_export. */
int hlq_weight_to_export(const hlq_weight *w, void *h_w_quant, void *h_w_scale, void *h_w_zero,
                         void *h_bias_or_null, void *stream);
/* Replaces: ~weight_tensor, C++/ops/include/arm/arm_nnstructures.h:30-36. */
int hlq_weight_free(hlq_weight *w);
int hlq_weight_get_info(const hlq_weight *w, hlq_weight_info *info);
/* Device pointers of the handle's buffers (NULL where the layout has none): the packed
 * planes, the scales/zeros, and the bias.  For benchmarks that fill weights on the device. */
int hlq_weight_buffers(const hlq_weight *w, void **d_planes, int64_t *planes_bytes,
                       void **d_meta, int64_t *meta_bytes, void **d_bias);
/* Allocate a weight of the given (unsharded) shape with undefined contents, to be filled
 * through hlq_weight_buffers.  No counterpart in the reference (benchmark helper). */
int hlq_weight_alloc(hlq_weight **out, int in_ch, int out_ch, int groupsize, int bits,
                     int has_bias, int device, unsigned flags);

/* The runtime's optional extra bit-plane ("sparse" weights, weight_config.json use_sparse = true): for a
 * list of blocks of 32 output rows x one group of input channels, one more bit-plane with one fp16 scale per
 * row, w[x + r, y + c] += scale[pair][r] * bit[pair][r][c].  h_mask: uint32 [pairs][2] = (first output row of
 * the block, first input channel of its group) in coordinates of the FULL weight; h_blocks: uint8
 * [pairs][32][g/8] (bit j of byte i = channel 8i+j of the group); h_scales: fp16 [pairs][32].  A sharded handle
 * keeps the blocks of its shard.  hlq_linear_forward then includes the plane (exactly for the LUT GEMV, which
 * takes it into its fp32 accumulators; as an addition to y after the other kernels); the grouped, fused
 * all-reduce, static-scratch and chain entry points refuse such weights (HLQ_ERR_UNSUPPORTED).
 * hlq_weight_get_sparse returns the kept blocks in the shard's coordinates (buffers sized by
 * hlq_weight_sparse_pairs).  Synchronize `stream`.
 * Replaces: the use_sparse branch of load_Parameter (C++/ops/src/arm/parameters.cpp:44-64), the re-layout
 * t_mac_g4_rearrange_weight_sparse_impl (C++/ops/src/arm/arm_t_mac_kernal.cpp:554-646) and the kernel
 * t_mac_g4_float_update_sparse_impl (arm_t_mac_kernal.cpp:678-788) with its drivers (arm_gemm.cpp:390-563). */
int hlq_weight_set_sparse(hlq_weight *w, const uint32_t *h_mask, int pairs, const uint8_t *h_blocks,
                          const uint16_t *h_scales, void *stream);
int hlq_weight_sparse_pairs(const hlq_weight *w, int *pairs);
int hlq_weight_get_sparse(const hlq_weight *w, uint32_t *h_mask, uint8_t *h_blocks, uint16_t *h_scales,
                          void *stream);

/* Optional: a second copy of the planes of a 2- or 3-bit weight in the streaming layout as one 4-bit
 * code word per weight (the planes' bits of a weight side by side; n_pad * k_pad / 2 bytes of device
 * memory, counted in hlq_weight_info.device_bytes).  Calls with 3..16 rows of activations then read
 * the code words instead of the planes and skip the bit gathering that binds them (their results
 * are the same numbers).  For g = 128 and rows a multiple of 128 the call also stores the codes a
 * third time with one row per lane ("row codes", as many bytes again plus 8 bytes per group), which
 * only the kernel that hlq_select_batch_kernel(3) selects reads.  Build it before the weight is put
 * into a group; it is freed with the handle and never exported.  No counterpart in the reference. */
int hlq_weight_build_batch_codes(hlq_weight *w, void *stream);

/* ---- forward ------------------------------------------------------------------------ */

/* Bytes of device scratch hlq_linear_forward needs for this problem (0 is possible).
 * Replaces the temp_workplace sizing of C++/ops/src/arm/arm_gemm.cpp:333-334,348.
 * A workspace sized for m rows serves every call with at most m rows, in any order: the regions
 * of the kernels do not overlap (status word; counters and fp32 accumulators of the 1..16-row
 * kernels, zero between calls; above 16 rows an fp16 copy of bf16 activations and, up to 256
 * rows, fp32 slabs [m][n] for problems that are split along K).  After a call that ended with
 * HLQ_ERR_KERNEL zero the workspace again (hlq_workspace_init). */
size_t hlq_workspace_bytes(int m, int k, int n, int bits, int groupsize);
/* Zero a freshly allocated workspace once, before its first use (the forward kernels
 * leave it in the state they need).  One workspace serves one stream at a time. */
int hlq_workspace_init(void *d_workspace, size_t bytes, void *stream);

/* Read the status word the kernels of the last launches left in the workspace
 * (synchronizes `stream`).  Returns HLQ_ERR_KERNEL and a non-zero *kernel_status when a
 * kernel gave up on a bounded wait (1) or found its shared-memory window unusable (2).
 * No counterpart in the reference, whose CPU kernel has no asynchronous failures. */
int hlq_workspace_status(const void *d_workspace, void *stream, int *kernel_status);

/* y[m, n] = x[m, k] . W_hat^T + bias, W_hat = sum_i alpha_i b_i + z; y is overwritten.
 * x and y are device pointers with row strides k and n; x_dtype in {F16, BF16}, y_dtype in
 * {F16, BF16, F32}; accumulation is fp32.  k and n must equal the handle's shard sizes.
 * With HLQ_SHARD_COLS the result is this rank's partial sum.  Not re-entrant on one
 * workspace.  x and y must be 16-byte aligned.
 * Kernels by m (streaming layout): 1 or 2 rows, and fp32 outputs up to 16 rows: table-lookup
 * GEMV; 3..16 rows with 16-bit outputs at 2 or 3 bits: one pass over the weights for all rows
 * (dequantization in registers + mma.sync; the weights are rounded to fp16 there); more rows:
 * dequantization + tcgen05 GEMM.
 * Replaces: arm_gemm, C++/ops/include/arm/arm_gemm.h:4-14 (dispatch at
 * C++/ops/src/arm/arm_gemm.cpp:871-924; GEMV worker :248-308, GEMM worker :362-387). */
int hlq_linear_forward(int m, int k, int n, const void *d_x, int x_dtype, void *d_y, int y_dtype,
                       void *d_workspace, size_t workspace_bytes, const hlq_weight *w,
                       void *stream);

/* Same contract, but forces one implementation: 0 = automatic (what hlq_linear_forward
 * does), 1 = LUT GEMV on the streaming layout, 2 = generic LUT GEMV on the exported layout,
 * 3 = dequantize + tensor-core GEMM.  For tests and measurements. */
int hlq_linear_forward_impl(int impl, int m, int k, int n, const void *d_x, int x_dtype,
                            void *d_y, int y_dtype, void *d_workspace, size_t workspace_bytes,
                            const hlq_weight *w, void *stream);

/* Which kernel serves 3..16 rows of activations (for tests and measurements, process-wide):
 * 0 = the default (1), 1 = register dequantization + mma.sync, 2 = register dequantization +
 * tcgen05.mma with the weight operand in shared memory and the accumulators in tensor memory
 * (correct, the slowest of the three), 3 = tcgen05.mma with the weight operand in tensor memory
 * (needs the row codes that hlq_weight_build_batch_codes makes for 2- and 3-bit weights with
 * g = 128 and rows a multiple of 128; other weights fall back to 1; as fast as 1 at 16 rows,
 * slower below).  Same results up to fp32 summation order. */
int hlq_select_batch_kernel(int which);

/* Which kernel serves more than 16 rows of activations (for tests and measurements,
 * process-wide): 0 = the default (2), 1 = one CTA per tile of 256 (128) weight rows, both operands
 * in shared memory, 2 = a pair of CTAs per tile of 256 weight rows, persistent over the tiles, the
 * dequantized weights in tensor memory, the token tile shared by the pair.  Same results up to
 * fp32 summation order. */
int hlq_select_prefill_kernel(int which);

/* The same product as hlq_linear_forward for a weight in the streaming layout, for callers
 * that must not allocate device memory around the call and therefore have no workspace to
 * pass: a serving process whose own memory manager took all of HBM at start-up, or a
 * latency-critical section that cannot tolerate the device-wide synchronization of
 * cudaMalloc/cudaFree.  The scratch (status word, completion counters, fp32 accumulators)
 * lives in a fixed HLQ_STATIC_SCRATCH_BYTES array inside the library, which every GPU that
 * loads the library holds until the process exits.  The call allocates nothing.
 *  - Limit: the scratch of one launch, 256 + 4 * r * ceil(n/32) (rounded up to 256) +
 *    4 * r8 * 32 * ceil(n/32) bytes with r = min(m, 16) rows per launch and r8 = r rounded up to
 *    8 when r >= 2 (more rows run as several launches of 16), must fit
 *    HLQ_STATIC_SCRATCH_BYTES, else HLQ_ERR_WORKSPACE (m = 1: n up to ~250 000 rows;
 *    m >= 9: n up to ~15 000).  Weights in the exported
 *    layout: HLQ_ERR_UNSUPPORTED.
 *  - The first call on a device looks the array's address up (with the weight's device
 *    current, as for hlq_linear_forward); make that first call before any stream capture.
 *  - All calls on a device share the one array.  Each call clears the counters and
 *    accumulators it uses on `stream` before its kernel, so leftovers of earlier calls do not
 *    matter, but two calls whose work overlaps on the GPU (different streams) race on it:
 *    keep them on one stream or order them with events.
 *  - The kernels' status word is the first word of the array.  The forward calls never clear
 *    it; hlq_static_scratch_status reads it (synchronizing `stream`), clears it, and returns
 *    HLQ_ERR_KERNEL with a non-zero *kernel_status exactly as hlq_workspace_status does, so a
 *    failure of any call since the last look is reported.  `device` must be current.
 * These entry points have no counterpart in the reference (its CPU operator gets its
 * temp_workplace from the caller, arm_gemm.h:4-14). */
#define HLQ_STATIC_SCRATCH_BYTES (1u << 20)
int hlq_linear_forward_static(int m, int k, int n, const void *d_x, int x_dtype, void *d_y,
                              int y_dtype, const hlq_weight *w, void *stream);
int hlq_static_scratch_status(int device, void *stream, int *kernel_status);

/* ---- groups: many independent linears in one launch ----------------------------------- */

/* A group runs the GEMVs of `count` loaded weights (all with the streaming layout, the same
 * bits and group size, on one device) as ONE persistent kernel launch: the CTAs walk the
 * concatenated work of all members, so small projections cost no launch of their own.  The
 * members must be independent: no y may alias an x of the same group.  The group owns its
 * scratch (per member: completion counters and per-slice partial sums for up to max_m rows,
 * max_m <= 16) and does not own the weights, which must outlive it.
 * Replaces the per-projection arm_gemm calls of one decoder layer,
 * C++/examples/models/llama.cpp:244-675, for projections whose inputs are ready together. */
typedef struct hlq_group hlq_group;
int hlq_group_create(hlq_group **out, int count, const hlq_weight *const *weights, int max_m);
/* Set the activation and output pointers of every member (host arrays of `count` device
 * pointers, x[i] = [m, k_i] 16-byte aligned, y[i] = [m, n_i]); synchronizes `stream`.  The
 * binding stays until the next call, so that hlq_group_forward is a bare kernel launch. */
int hlq_group_bind(hlq_group *g, const void *const *d_x, void *const *d_y, int x_dtype,
                   int y_dtype, void *stream);
/* y_i[m, n_i] = x_i[m, k_i] . W_hat_i^T + bias_i for every member, m <= max_m. */
int hlq_group_forward(hlq_group *g, int m, void *stream);
/* Status word of the group's kernels, as hlq_workspace_status. */
int hlq_group_status(const hlq_group *g, void *stream, int *kernel_status);
int hlq_group_info(const hlq_group *g, int *count, int64_t *scratch_bytes,
                   int64_t *algorithmic_bytes);
int hlq_group_free(hlq_group *g);

/* ---- tensor parallelism: GEMV with the all-reduce fused into its epilogue ---------------- */

/* A communicator owns, on every rank, a receive buffer that all ranks of the node map into
 * their address space (CUDA IPC over NVLink).  hlq_linear_forward_allreduce runs a
 * row-parallel (HLQ_SHARD_COLS) linear and sums the ranks' outputs inside the same kernel:
 * as soon as a rank has finished a block of 32 output rows it stores the block's sums into
 * every rank's buffer and raises a flag there; at its end every CTA waits (bounded) for the
 * flags of its share of blocks and adds the ranks' sums in rank order, so all ranks write the
 * same y.  No separate collective is launched.  Every rank must make the same sequence of
 * calls on one communicator; one communicator serves one stream.  world <= 8, one process per
 * GPU.  No counterpart in the reference, which has no multi-device path. */
typedef struct hlq_tp_comm hlq_tp_comm;
int hlq_tp_comm_create(hlq_tp_comm **out, int rank, int world, int max_n, int max_m, int device);
/* 64 opaque bytes that the other ranks need (exchange them with any host-side all-gather). */
int hlq_tp_comm_handle(const hlq_tp_comm *c, void *handle64);
/* handles: world x 64 bytes, in rank order (this rank's own entry is ignored). */
int hlq_tp_comm_connect(hlq_tp_comm *c, const void *handles);
/* The same connection for ranks that live in ONE process (one thread per GPU with peer access
 * enabled, or a test that stands in for an absent peer with a buffer nobody writes):
 * d_peer_buffers[p] is rank p's receive buffer (hlq_tp_comm_local_buffer of its communicator,
 * or any zeroed, 256-byte aligned device allocation of hlq_tp_comm_buffer_bytes bytes) as
 * addressable from this rank's device; this rank's own entry is ignored. */
int hlq_tp_comm_buffer_bytes(const hlq_tp_comm *c, size_t *bytes);
int hlq_tp_comm_local_buffer(const hlq_tp_comm *c, void **d_buffer);
int hlq_tp_comm_connect_pointers(hlq_tp_comm *c, void *const *d_peer_buffers);
/* Polls after which a wait for a peer gives up (default 2^22, a few seconds).  The first
 * wait of a CTA that runs out makes all its later waits give up at once, the kernel ends
 * within microseconds of that, and the workspace status word reads 1.  After such a failure
 * the ranks' launch numbers no longer agree: free the communicator and create a new one. */
int hlq_tp_comm_set_spin_limit(hlq_tp_comm *c, int polls);
int hlq_tp_comm_free(hlq_tp_comm *c);
/* As hlq_linear_forward for m <= max_m rows and a streaming-layout weight; y receives the sum
 * over all ranks.  A rank that never arrives makes the others give up after a bounded wait
 * and report through the workspace status word (hlq_workspace_status returns HLQ_ERR_KERNEL
 * with *kernel_status == 1). */
int hlq_linear_forward_allreduce(int m, int k, int n, const void *d_x, int x_dtype, void *d_y,
                                 int y_dtype, void *d_workspace, size_t workspace_bytes,
                                 const hlq_weight *w, hlq_tp_comm *comm, void *stream);

/* ---- input transforms fused into the LUT GEMV ------------------------------------------
 *
 * The GEMV reads its activations slice by slice to build its lookup tables; an elementwise
 * op (or a norm) in front of a linear can be applied right there instead of in a kernel of
 * its own.  fp16 activations, streaming-layout weights, m <= 16 (one row of x per pass).
 *   HLQ_INPUT_GATED_SILU:  x_eff = fp16(second * x / (1 + exp(-x)))       x = gate, second = up
 *       = gated_silu (C++/ops/src/arm/arm_activation.cpp:22-52) in front of down_proj
 *   HLQ_INPUT_ADD_RMSNORM: t = x + second (second may be NULL); res_out = fp16(t) (may be
 *       NULL, must not alias x or second); x_eff = fp16(fp16(t) * gamma / sqrt(mean(t^2) + eps))
 *       = launch_pre_rms_norm / launch_rms_norm (C++/ops/src/arm/arm_rmsnorm.cpp:25-41, 68-85)
 *       in front of q/k/v, gate/up or lm_head.
 * The values the tables see are rounded to fp16 exactly where the separate kernels
 * (hlq_gated_silu, hlq_rmsnorm) round. */
typedef enum hlq_input_kind {
    HLQ_INPUT_PLAIN = 0,
    HLQ_INPUT_GATED_SILU = 1,
    HLQ_INPUT_ADD_RMSNORM = 2
} hlq_input_kind;
typedef struct hlq_input_op {
    int kind;               /* hlq_input_kind */
    float eps;              /* ADD_RMSNORM */
    const void *d_second;   /* fp16 [m][k] */
    const void *d_gamma;    /* ADD_RMSNORM: fp16 [k] */
    void *d_res_out;        /* ADD_RMSNORM: fp16 [m][k] or NULL */
} hlq_input_op;
/* hlq_linear_forward with an input transform (op NULL or PLAIN: the same as hlq_linear_forward
 * restricted to the LUT GEMV). */
int hlq_linear_forward_op(int m, int k, int n, const void *d_x, int x_dtype, void *d_y, int y_dtype,
                          void *d_workspace, size_t workspace_bytes, const hlq_weight *w,
                          const hlq_input_op *op, void *stream);
/* hlq_linear_forward_allreduce with an input transform. */
int hlq_linear_forward_allreduce_op(int m, int k, int n, const void *d_x, int x_dtype, void *d_y,
                                    int y_dtype, void *d_workspace, size_t workspace_bytes,
                                    const hlq_weight *w, hlq_tp_comm *comm, const hlq_input_op *op,
                                    void *stream);
/* hlq_group_bind with one input transform per member (ops NULL: none).  Members that share an
 * ADD_RMSNORM input should name d_res_out in one of them only. */
int hlq_group_bind_op(hlq_group *g, const void *const *d_x, void *const *d_y, int x_dtype,
                      int y_dtype, const hlq_input_op *ops, void *stream);

/* ---- decoder glue between the linears (fp16, device pointers, one token) --------------
 *
 * The per-token ops the reference's model runs between two quantized linears
 * (C++/examples/models/llama.cpp:193-215, 396-476, 554, 646, 717, 763).  All pointers are
 * device pointers to fp16 unless noted, 16-byte aligned; all work is queued on `stream`. */

/* out[r,:] = t * gamma / sqrt(mean(t^2) + eps), t = x[r,:] (+ residual[r,:]).  With a
 * residual, t is also stored rounded to fp16 in res_out and the rounded value is what gets
 * normalized.  out may alias x and res_out may alias residual (the reference calls it so).
 * n % 8 == 0.  Replaces launch_rms_norm / launch_pre_rms_norm
 * (C++/ops/src/arm/arm_rmsnorm.cpp:165-212; math at :25-41 and :68-85). */
int hlq_rmsnorm(int rows, int n, const void *d_x, const void *d_residual_or_null,
                void *d_res_out_or_null, const void *d_gamma, float eps, void *d_out, void *stream);

/* out = up * gate / (1 + exp(-gate)) in fp32, rounded to fp16; rows * n % 8 == 0.  Replaces
 * gated_silu (C++/ops/src/arm/arm_activation.cpp:22-52, 92-106). */
int hlq_gated_silu(int rows, int n, const void *d_gate, const void *d_up, void *d_out, void *stream);

/* Index (and optionally value) of the first largest of n values (dtype HLQ_F16 or HLQ_F32).
 * Replaces arm_argmax_last for one token (C++/ops/src/arm/arm_argmax.cpp:3-29). */
int hlq_argmax(int n, const void *d_values, int dtype, int *d_index_out, float *d_value_out_or_null,
               void *stream);

/* One decode step of attention for one token, in one kernel:
 *   RoPE on q [head_q][dhead] and k [head_kv][dhead] with pairs (j, j + dhead/2) and angle
 *   position * rotary_base^(-2j/dhead)      (launch_llama_qkv_apply_rotary, arm_rotary.cpp:4-88),
 *   append of the roped k and of v at `position` into the caches (layout: hlq_kv_layout)
 *                                           (arm_cache, arm_cache.cpp:3-22),
 *   softmax(scale * q.K) V over positions 0..position with head h reading kv head
 *   h * head_kv / head_q                    (arm_attention, arm_attention.cpp:196-270, 320-340).
 * `d_position` points to ONE int in device memory (so a captured graph can be replayed for
 * the next token after the caller increments it); a position outside [0, max_ctx) is clamped
 * and reported through the workspace status word (hlq_workspace_status).  dhead 64 or 128,
 * head_q / head_kv <= 8.  The workspace needs hlq_attention_workspace_bytes(...) bytes, zeroed
 * once with hlq_workspace_init; one workspace per stream. */
typedef enum hlq_kv_layout {
    HLQ_KV_POSITION_MAJOR = 0, /* [max_ctx][head_kv][dhead], the reference's caches (arm_cache.cpp:17-21)  */
    HLQ_KV_HEAD_MAJOR = 1      /* [head_kv][max_ctx][dhead]: a head's positions are contiguous, which is    */
                               /* what a GPU wants (a CTA reads 32 KB runs instead of 256 B every 2 KB)   */
} hlq_kv_layout;
size_t hlq_attention_workspace_bytes(int head_q, int head_kv, int dhead, int max_ctx);
int hlq_rope_cache_attention(const void *d_q, const void *d_k, const void *d_v, void *d_kcache,
                             void *d_vcache, const int *d_position, int head_q, int head_kv,
                             int dhead, int max_ctx, int kv_layout, float rotary_base, float scale,
                             void *d_out, void *d_workspace, size_t workspace_bytes, void *stream);

/* ---- decode chain: one token's ops of all layers as one persistent kernel ----------------
 *
 * The reference's model runs one call per op and token (C++/examples/models/llama.cpp:185-700:
 * per layer RMSNorm, q/k/v, RoPE, cache append, attention, o, residual add + RMSNorm, gate/up,
 * gated SiLU, down).  A chain is that list of ops recorded once and then run, for every token,
 * by ONE kernel whose CTAs stay resident: a STAGE is a set of linears whose inputs are ready
 * together (hlq_chain_add_linears) or the attention of one token (hlq_chain_add_attention);
 * stage s + 1 starts reading when stage s has written everything (a counter in device memory,
 * polled with a bounded wait).  The elementwise ops sit in the linears:
 *   input   HLQ_CHAIN_IN_PLAIN     x = the fp16 activations [k];
 *           HLQ_CHAIN_IN_NORM      x = the residual stream [k]; the tables are built from
 *                                  fp16(x * gamma / sqrt(cell[ss_in] / norm_channels + eps)),
 *                                  where the cell was filled by the stage that last updated the stream
 *                                  (launch_rms_norm / launch_pre_rms_norm, arm_rmsnorm.cpp:25-41, 68-85);
 *           HLQ_CHAIN_IN_ATTENTION x = the output of the attention stage recorded just before (d_x is
 *                                  ignored): the attention units leave one partial result per split of the
 *                                  context, and this linear merges them while it loads its activations
 *                                  (the merge of arm_attention.cpp:320-340's per-head results, without a pass
 *                                  or a hand-off of its own); k must be head_q * 128;
 *   output  HLQ_CHAIN_OUT_STORE    y[n] = fp16(result);
 *           HLQ_CHAIN_OUT_RESIDUAL y is the residual stream: t = y + fp16(result), y = fp16(t),
 *                                  cell[ss_out] += sum t^2                  (arm_rmsnorm.cpp:68-85);
 *           HLQ_CHAIN_OUT_GATED_SILU the weight's rows alternate in chunks of 16 between gate rows
 *                                  and up rows (rows 32c..32c+15 = gate 16c..16c+15, rows 32c+16..32c+31
 *                                  = up 16c..16c+15); y[n/2] = fp16(up * gate / (1 + exp(-gate)))
 *                                  (gated_silu, arm_activation.cpp:36-49).
 * With a communicator (one linear per stage, HLQ_SHARD_COLS weight) the ranks' results are summed
 * inside the kernel before the output op, as in hlq_linear_forward_allreduce; every rank must
 * record the same chain.  All members share bits and group size, use the streaming layout and
 * fp16 activations, batch 1.  The chain owns its scratch; weights, buffers and the communicator
 * must outlive it.  hlq_chain_forward clears the chain's counters on `stream` and launches the
 * kernel (no allocation; it can be captured into a CUDA graph).  hlq_chain_status reads the
 * status word (1: a wait ran out, 2: shared-memory window unusable) as hlq_workspace_status does. */
typedef struct hlq_chain hlq_chain;
typedef enum hlq_chain_in { HLQ_CHAIN_IN_PLAIN = 0, HLQ_CHAIN_IN_NORM = 1, HLQ_CHAIN_IN_ATTENTION = 2 } hlq_chain_in;
typedef enum hlq_chain_out {
    HLQ_CHAIN_OUT_STORE = 0,
    HLQ_CHAIN_OUT_RESIDUAL = 1,
    HLQ_CHAIN_OUT_GATED_SILU = 2
} hlq_chain_out;
typedef struct hlq_chain_linear {
    const hlq_weight *w;
    const void *d_x;      /* fp16 [k], 16-byte aligned */
    void *d_y;            /* fp16: [n], the residual stream [n], or [n/2] (see hlq_chain_out) */
    int in_kind;          /* hlq_chain_in */
    int out_kind;         /* hlq_chain_out */
    const void *d_gamma;  /* IN_NORM: fp16 [k], 16-byte aligned */
    float eps;            /* IN_NORM */
    int norm_channels;    /* IN_NORM: channels the sum of squares covers (0: k) */
    int ss_in;            /* IN_NORM: cell to read */
    int ss_out;           /* OUT_RESIDUAL: cell to accumulate into */
} hlq_chain_linear;
int hlq_chain_create(hlq_chain **out, int device, int ss_cells);
int hlq_chain_add_linears(hlq_chain *c, int count, const hlq_chain_linear *members, hlq_tp_comm *comm_or_null);
/* Arguments as hlq_rope_cache_attention (dhead 128 only; all attention stages of a chain share d_position,
 * rotary_base and max_ctx).  d_out is written only by hlq_rope_cache_attention: in a chain the stage's
 * result is consumed by the next stage's linear through HLQ_CHAIN_IN_ATTENTION. */
int hlq_chain_add_attention(hlq_chain *c, const void *d_q, const void *d_k, const void *d_v, void *d_kcache,
                            void *d_vcache, const int *d_position, int head_q, int head_kv, int dhead,
                            int max_ctx, int kv_layout, float rotary_base, float scale, void *d_out,
                            void *d_workspace, size_t workspace_bytes);
/* Ends the recording: allocates the scratch and uploads the tables (synchronizes `stream`). */
int hlq_chain_finish(hlq_chain *c, void *stream);
int hlq_chain_forward(hlq_chain *c, void *stream);
int hlq_chain_status(const hlq_chain *c, void *stream, int *kernel_status);
/* Profiling aid: with a device buffer of ctas x items_per_cta x 16 uint64 (zeroed by the caller), the
 * next forwards write a timeline into it: for item i of CTA c, entry [c][i][k] is the nanosecond clock when
 * (k = 0) the control warp saw the item's gate open, (1) had issued its input copies, (2, 3) the consumers
 * began and ended waiting for the inputs, (4) agreed to run, (5) had built the tables, (6) ended streaming,
 * (7) handed the item over, (8, 9, 10) the finalizers took it, had published it, had summed the ranks.
 * d_trace NULL or items_per_cta 0 turns it off.  *ctas receives the grid size. */
int hlq_chain_trace(hlq_chain *c, void *d_trace, int items_per_cta, int *ctas);
int hlq_chain_info(const hlq_chain *c, int *stages, int *linears, int *rank_sums, int64_t *scratch_bytes);
int hlq_chain_free(hlq_chain *c);

/* ---- diagnostics -------------------------------------------------------------------- */

/* Human-readable text for an hlq_status.  Replaces the reference's exit(-1)/exceptions
 * (C++/common/include/Allocate.h:10-13, C++/common/src/fileutils.cpp:32-43). */
const char *hlq_last_error_string(int status);
/* cudaError_t of the most recent failing CUDA call on this thread (0 if none). */
int hlq_last_cuda_error(void);
/* Number of kernels this library has launched in this process (all threads). */
int64_t hlq_kernel_launch_count(void);
/* ABI version of this header. */
int hlq_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* HLQ_B200_H */
