/*
 * spiky_b200 - C ABI of the B200-native LUT-layer runtime.
 *
 * Every entry point takes raw device pointers, sizes and a CUDA stream handle and returns an int
 * status: 0 = ok, < 0 = argument error (LUTB_ERR_*), > 0 = a cudaError_t raised by a launch.
 * Nothing throws, aborts or allocates unless stated.  lutb_last_error() returns a thread-local,
 * human readable description of the last non-zero status.
 *
 * The functions replace the runtime methods of the reference's pybind11 classes
 * LUTDataManagerF / LUTDataManagerI (registered in spiky_cuda/spiky_py.cpp:6-24, defined in
 * spiky_cuda/lut/lut.cu); each declaration cites the method it stands in for.  Tensor layouts are
 * the reference's: all arrays flat, contiguous, fp32 / int32, outputs accumulated into
 * caller-zeroed buffers.  Unlike the reference, kernels are enqueued on ONE caller-supplied stream
 * and the call returns without synchronising.
 */
#ifndef SPIKY_B200_H
#define SPIKY_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LUTB_OK 0
#define LUTB_ERR_NULL (-1)      /* a required pointer is NULL */
#define LUTB_ERR_SHAPE (-2)     /* a size is zero, negative or out of the supported range */
#define LUTB_ERR_MODE (-3)      /* inconsistent flags (e.g. dW given together with an internal learning rate) */
#define LUTB_ERR_WORKSPACE (-4) /* workspace missing or too small */
#define LUTB_ERR_ALIGN (-5)     /* a pointer is not aligned as documented */

/* weight-gradient kernel selection for the backward entry points */
#define LUTB_DW_AUTO 0      /* the library's choice between the two below by measured contention: on B200 ATOMIC won at every
                               point of the sweep (0.06 to 4096 samples per table row, 2.3x to 10x), so AUTO is ATOMIC */
#define LUTB_DW_ATOMIC 1    /* row-coalesced global reductions (red.global.add.v4.f32 into L2) */
#define LUTB_DW_SORTED 3    /* counting sort of the batch by row + segmented reduce; deterministic order; needs workspace */

/*
 * Geometry and numeric mode of one LUT layer; mirrors the constructor arguments of
 * LUTDataManagerF/I (spiky_cuda/lut/lut.cu:17-31) plus the per-call scalars.
 */
typedef struct lutb_layer_cfg {
    int32_t n_inputs;        /* I  */
    int32_t n_outputs;       /* O  */
    int32_t n_detectors;     /* Nt */
    int32_t n_anchors;       /* Nc, 1..30; a table has 2^Nc rows (non-sequence and product layers) */
    int32_t seq_len;         /* S, 1 for non-sequence layers */
    int32_t pos_dim;         /* Npe, 0 when unused */
    int32_t forward_group;   /* forward_group_size: outputs per block in the backward pass */
    int32_t backward_group;  /* backward_group_size: detectors per block in the forward pass */
    int32_t int_mode;        /* 0: fp32 accumulators (LUTDataManagerF); 1: int32 fixed point (LUTDataManagerI) */
    int32_t sliced_product;  /* product layers only: interleaved [x_i, x_j, pe] anchor numbering */
    float cmp_eps;           /* dead band of the anchor comparison, 0 = plain '>' */
    float reserved0;
    double int_rescaler;     /* fixed-point scale multiplier (int_mode == 1) */
    double lr_meta;          /* SynapseMeta.learning_rate applied to weight gradients */
} lutb_layer_cfg;

/* Library / build identification. */
int lutb_version(void);
const char *lutb_last_error(void);

/*
 * Opt-in kernel profiler.  Stands in for LUTDataManager::get_profiling_stats / reset_profiler
 * (spiky_cuda/lut/lut.cu:1274-1288; SimpleProfiler, spiky_cuda/misc/misc.h:365-405), which in the
 * reference is always on and synchronises the stream after every launch.  Here launches are only
 * counted by default; after lutb_profiler_enable(1) each launch is additionally bracketed by CUDA
 * events on its stream, resolved lazily by lutb_profiler_read (which waits for the recorded events).
 * Kernel ids run from 0 to lutb_profiler_kernel_count() - 1.
 */
int lutb_profiler_enable(int on);
int lutb_profiler_reset(void);
int lutb_profiler_kernel_count(void);
const char *lutb_profiler_kernel_name(int kernel_id);
int lutb_profiler_read(int kernel_id, double *total_ms, int64_t *timed_launches, int64_t *launches);

/*
 * Non-sequence, fully connected forward.  Replaces LUTDataManager::forward_step
 * (spiky_cuda/lut/lut.cu:629-716 -> LUTRuntimeContext::forward_step, lut_runtime.cu:76-211).
 *   weights    fp32 [Nt * 2^Nc * O]        anchors  int32 [Nt * Nc * 2] (-1 = unused pair)
 *   x          fp32 [batch * I]            y        fp32 [batch * O], accumulated into
 *   idx        int32 [batch * Nt] out      min_delta fp32 / min_k int32 [batch * Nt] out, both NULL = eval
 */
int lutb_nonseq_fc_forward(const lutb_layer_cfg *cfg, int64_t batch, const float *weights, const float *x,
                           const int32_t *anchors, float *y, int32_t *idx, float *min_delta, int32_t *min_k,
                           void *stream);

/*
 * Bytes of scratch memory lutb_nonseq_fc_backward needs for the given variant (0 for all but
 * LUTB_DW_SORTED).  The caller allocates it; 256-byte alignment is required.
 */
size_t lutb_nonseq_fc_backward_workspace(const lutb_layer_cfg *cfg, int64_t batch, int dw_variant);

/*
 * Non-sequence, fully connected backward.  Replaces LUTDataManager::backward_backprop
 * (spiky_cuda/lut/lut.cu:1030-1088 -> LUTRuntimeContext::backward_backprop, lut_runtime.cu:213-397).
 *   dX  fp32 [batch * I] accumulated into; NULL (not possible in the reference, which always computes it) skips
 *       the input-gradient kernels: for a first layer whose input needs no gradient.
 *   external_lr < 0: dW fp32 [Nt * 2^Nc * O] receives lr_meta * dY rows (accumulated into).
 *   external_lr >= 0: dW must be NULL and weights are updated in place by -external_lr * lr_meta * dY.
 *   external_lr == LUTB_SKIP_TABLE_GRADIENT (-2.0, dW must be NULL): only the input gradient; the caller takes the
 *       table gradient in another form (lutb_nonseq_fc_table_grad_rows).
 */
int lutb_nonseq_fc_backward(const lutb_layer_cfg *cfg, int64_t batch, float *weights, const float *dY,
                            const int32_t *anchors, const int32_t *idx, const float *min_delta,
                            const int32_t *min_k, float *dX, float *dW, double external_lr, int dw_variant,
                            void *workspace, size_t workspace_bytes, void *stream);

/*
 * Table gradient of a non-sequence, fully connected layer as a list of touched rows, for the Sparse gradient policy.
 * The reference forms the dense gradient and compacts it afterwards (LUTLayerBasic._process_gradients,
 * src/spiky/lut/LUTLayer.py:567-609 -> DenseToSparseConverterNative, spiky_cuda/torch_utils/torch_utils.cu:29-322); a
 * step touches at most batch rows per detector, so here the list comes straight from the table-gradient pass and
 * nothing of the size of the tables is written or read:
 *   row_ids int64 [capacity]           detector * 2^Nc + row of every touched row, ascending
 *   values  fp32  [capacity * O]       the row's gradient: lr_meta * sum over the samples that selected it of dY[b, :]
 *                                      (|dY| > 1e-17), samples added in ascending order (as LUTB_DW_SORTED does)
 *   count_out int64 (device)           number of touched rows; rows beyond capacity are counted, not written
 * capacity >= min(batch, 2^Nc) * Nt always suffices.  fp32 accumulators only; the workspace (256-byte aligned) must
 * hold lutb_nonseq_fc_table_grad_rows_workspace(cfg, batch) bytes.
 */
size_t lutb_nonseq_fc_table_grad_rows_workspace(const lutb_layer_cfg *cfg, int64_t batch);
int lutb_nonseq_fc_table_grad_rows(const lutb_layer_cfg *cfg, int64_t batch, const float *dY, const int32_t *idx,
                                   int64_t *row_ids, float *values, int64_t capacity, int64_t *count_out,
                                   void *workspace, size_t workspace_bytes, void *stream);

/*
 * Non-sequence, fully connected backward for callers that must not allocate device memory.
 * No counterpart in the reference (its runtime allocates through torch at every call).
 *
 * Who needs it: code that runs where cudaMalloc is unavailable or forbidden - inside a host callback or a
 * real-time loop that may not block on the allocator, in a process whose memory pool is owned and fully
 * handed out by another component, or under a memory budget that was fixed at start-up.  Such a caller
 * cannot provide the workspace that lutb_nonseq_fc_backward(..., LUTB_DW_SORTED, workspace, ...) wants.
 *
 * This entry point computes exactly what that call computes (deterministic table gradient: per cell the
 * samples are added in ascending order; fp32 accumulators only, cfg->int_mode must be 0) but takes its
 * scratch from an array of LUTB_STATIC_SCRATCH_BYTES bytes that is part of the library's device image.  It
 * calls no cudaMalloc / cudaFree and no allocating library routine, and it records no profiler events.
 *   - limit: lutb_nonseq_fc_backward_workspace(cfg, batch, LUTB_DW_SORTED) must not exceed
 *     LUTB_STATIC_SCRATCH_BYTES; larger problems are refused with LUTB_ERR_WORKSPACE and a message;
 *   - the first call on a device looks the array's device address up (cudaGetSymbolAddress with that device
 *     current); make that first call before any stream capture begins.  Like any first launch it may also make the CUDA runtime
 *     load the library's module and kernels (lazy loading), which allocates inside the driver: call it once at
 *     start-up, before the phase that must not allocate;
 *   - every call on a device shares the one array and overwrites what the previous call left there (the part
 *     that must start at zero is cleared on the stream first): two calls that overlap on the GPU, e.g. on
 *     different streams, race; serialise them;
 *   - every GPU that loads the library carries the array for the life of the process.
 * Arguments as lutb_nonseq_fc_backward without dw_variant / workspace.
 */
#define LUTB_STATIC_SCRATCH_BYTES (8u << 20)
int lutb_nonseq_fc_backward_noalloc(const lutb_layer_cfg *cfg, int64_t batch, float *weights, const float *dY,
                                    const int32_t *anchors, const int32_t *idx, const float *min_delta,
                                    const int32_t *min_k, float *dX, float *dW, double external_lr, void *stream);

/*
 * Sparse lookup -> output connectivity (projection / convolution layers), all arrays in device memory.
 * Stands in for the reference's forward-synapse-group arena (ForwardSynapseGroup runs per lookup neuron,
 * spiky_cuda/connections_manager/connections_manager.h:39-66, indexed through NoDelaysIndexedSynapsesInfo,
 * :124-131).  The lookup neurons (table rows) of one detector share one target list; the flat weight
 * array keeps the reference's slot layout: synapse p of a row at row_base + p + 2 * (p / group_size),
 * rows det_stride apart.
 */
typedef struct lutb_sparse_index {
    const int64_t *det_wbase;   /* [Nt] weight slot of (row 0, synapse 0) */
    const int32_t *det_stride;  /* [Nt] slots between consecutive rows */
    const int32_t *det_count;   /* [Nt] synapses per row */
    const int32_t *det_sstart;  /* [Nt] exclusive prefix sum of det_count */
    const int32_t *syn_det;     /* [n_syn_per_sample] detector of each (detector, synapse) pair, detector order */
    const int32_t *syn_target;  /* [n_syn_per_sample] output index of each pair */
    const int32_t *chunk_info;  /* [n_chunks][8], 32-byte aligned: first detector, detector count (<= 32), offset of
                                   the shared target list in syn_target, synapses per row, row stride, slots per
                                   detector table (rows * stride), det_wbase of the first detector (low, high
                                   word).  A chunk is a run of consecutive detectors with identical target lists
                                   whose tables lie back to back and together span < 2^31 slots */
    int64_t n_chunks;
    int64_t n_syn_per_sample;   /* sum of det_count */
    int64_t n_weights;          /* length of the flat weight array */
    int32_t group_size;         /* forward_group_size G */
    int32_t max_count;          /* max of det_count */
    int32_t max_table_slots;    /* largest "slots per detector table" of chunk_info; 0 = unknown (gather kernels only) */
    int32_t tables_aligned16;   /* 1 when every detector table starts at a multiple of 4 slots and spans a multiple of
                                   4 slots, so that it can be bulk-copied with 16-byte granularity; 0 otherwise */
} lutb_sparse_index;

/*
 * Kernel family of the forward pass and of the input-gradient pass of sparse non-sequence layers, chosen independently
 * (no reference counterpart: the reference has one kernel per pass).  Process-wide; the environment variable
 * LUTB_SPARSE_KERNELS="<forward>,<input gradient>" (or one word for both: auto, gather, staged) sets the initial value.
 *   GATHER  one warp per (detector chunk, few samples); the selected rows are fetched through L2.  Any layer.
 *   STAGED  a block owns a range of detectors for 512 samples at a time; whole tables are streamed through a
 *           shared-memory ring (cp.async.bulk + mbarrier) and the samples' rows are read from there.  fp32 accumulators,
 *           rows of at most 32 synapses, tables_aligned16, three tables must fit 227 KB; LUTB_ERR_MODE when forced and
 *           not possible.
 *   AUTO    forward: STAGED when possible, 2 * batch >= rows per table and the layer has at least 4 detectors per SM,
 *           else GATHER; input gradient: GATHER (the staged variant measured slower on B200).
 * lutb_device_wait_errors: every device-side wait (the staged kernels' and lutb_peer_barrier's) is bounded (about a
 * second); a wait that runs out makes its block leave early (results are then incomplete) and is counted here.  Reads the counter of the current
 * device and synchronises it; 0 in a healthy run.
 */
#define LUTB_SPARSE_AUTO 0
#define LUTB_SPARSE_GATHER 1
#define LUTB_SPARSE_STAGED 2
int lutb_sparse_kernel_select(int forward_kernels, int input_grad_kernels);
int lutb_device_wait_errors(int *count_out);

/*
 * Non-sequence, sparse forward.  Replaces LUTDataManager::forward_step for layers built with lookup
 * connections (lut.cu:629-716 -> fill_outputs_non_seq_sparse_logic, lut_runtime_kernels_logic.proto:1160-1212).
 * Arguments as lutb_nonseq_fc_forward; weights is fp32 [sp->n_weights].
 */
int lutb_nonseq_sparse_forward(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                               const float *weights, const float *x, const int32_t *anchors, float *y,
                               int32_t *idx, float *min_delta, int32_t *min_k, void *stream);

/*
 * Non-sequence, sparse backward.  Replaces LUTDataManager::backward_backprop for sparse layers
 * (lut.cu:1030-1088 -> propagate_through_detectors_non_seq_sparse_logic, proto:1303-1419, and
 * gather_w_gradients_non_seq_sparse_logic, proto:1501-1545).  Arguments as lutb_nonseq_fc_backward (dX may be
 * NULL).  Runs as two passes over the (sample, detector chunk) pairs: input gradient, then table gradient.
 * external_lr == LUTB_SKIP_TABLE_GRADIENT (dW must be NULL): only the input gradient; the caller makes the table
 * update itself with lutb_nonseq_sparse_table_grad.
 */
#define LUTB_SKIP_TABLE_GRADIENT (-2.0)
int lutb_nonseq_sparse_backward(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                float *weights, const float *dY, const int32_t *anchors, const int32_t *idx,
                                const float *min_delta, const int32_t *min_k, float *dX, float *dW,
                                double external_lr, void *stream);

/*
 * Table-gradient pass of a sparse non-sequence layer alone, over the detector chunks [chunk_begin, chunk_end) of
 * the index (lutb_sparse_index::chunk_info rows; a chunk is a run of up to 32 detectors with one target list):
 *   target[row(t, idx[b, t]) + p] += scale * cfg->lr_meta * dY[b, target(p)]   for |dY| > 1e-17,
 * the arithmetic of gather_w_gradients_non_seq_sparse_logic (lut_runtime_kernels_logic.proto:1501-1545).  target is
 * a dense gradient (scale 1) or the weights themselves (scale = -learning rate: in-place SGD).  No counterpart in
 * the single-process reference: it serves data-parallel ranks that each own a share of the detectors, gather
 * (idx, dY) of the whole batch - idx_bytes = 1 or 2 lets the indices travel as uint8 / uint16 when the tables have
 * at most 256 / 65536 rows - and update their share for all samples, instead of all-reducing dense gradients.
 *   idx  [batch * Nt] of idx_bytes-wide unsigned (4: int32) table indices; dY fp32 [batch * O].
 * fp32 accumulators only; rows of at most 32 synapses.
 */
int lutb_nonseq_sparse_table_grad(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                  const float *dY, const void *idx, int idx_bytes, float *target, double scale,
                                  int64_t chunk_begin, int64_t chunk_end, void *stream);

/*
 * Product-mode sequence layer, forward.  Replaces LUTDataManager::forward_step_product
 * (spiky_cuda/lut/lut.cu:847-943 -> LUTRuntimeContext::forward_step_product, lut_runtime.cu:852-1049).
 * For every causal pair i < j and detector t the table index is computed from
 * [x1[b,i,:] | x2[b,j,:] | pos_embeddings[j-i-1, t, :]] (cfg->sliced_product: interleaved numbering) and
 * row (t, index) is added to y[b, j, :].  Tables have 2^Nc rows.
 *   x1 fp32 [batch * seq_len * n_inputs_1], x2 likewise (the layer passes the same tensor twice)
 *   pos_embeddings fp32 [(seq_len - 1) * Nt * cfg->pos_dim] or NULL when cfg->pos_dim == 0
 *   anchors int32 [Nt * Nc * 2] over the virtual vector; y fp32 [batch * seq_len * O], accumulated into
 * cfg->seq_len and cfg->n_inputs are ignored (the reference builds the manager with sequence_length 1 and
 * n_inputs = 2 * E + pos_dim and passes the real sizes per call).  batch <= 65535, Nc <= 16.
 */
int lutb_product_forward(const lutb_layer_cfg *cfg, int64_t batch, int32_t seq_len, const float *weights,
                         const float *x1, const float *x2, int32_t n_inputs_1, int32_t n_inputs_2,
                         const float *pos_embeddings, const int32_t *anchors, float *y, int variant, void *workspace,
                         size_t workspace_bytes, void *stream);

/*
 * Kernel variants of the product-mode layer (no reference counterpart: the reference has one kernel per pass).
 *   DIRECT  one table row per (pair, detector) is gathered (forward) or gathered twice and scatter-added
 *           (backward) through L2; needs no workspace.
 *   HIST    per (query, detector) the selected rows are counted into a histogram first and the pass becomes dense
 *           contractions with the tables (see spiky_b200/csrc/product_hist.cuh): on the tensor cores when the library
 *           was built with them (lutb_fp32_gemm_available) and the workspace holds one sequence in their operand
 *           layout, else as register-tiled fp32 FMA contractions; fp32 accumulators only, 4 <= Nc <= 12, O % 4 == 0,
 *           16-byte aligned tensors, and a caller workspace of at least lutb_product_workspace(cfg, 1, S, backward)
 *           bytes (the batch is processed in chunks of as many sequences as fit); LUTB_ERR_WORKSPACE / LUTB_ERR_MODE
 *           when asked for and not possible.
 *   HIST_FMA  HIST with the fp32 FMA contractions forced.
 *   AUTO    HIST when it is possible, a workspace is supplied and the sequence is long enough against the
 *           table (4 * S >= 2^Nc; forward without tensor cores: S >= 2^Nc), else DIRECT.
 * lutb_product_workspace returns the bytes that let `batch` sequences go through in one chunk.
 */
#define LUTB_PRODUCT_AUTO 0
#define LUTB_PRODUCT_DIRECT 1
#define LUTB_PRODUCT_HIST 2
#define LUTB_PRODUCT_HIST_FMA 3
/*
 * Flags or'ed into `variant` (training: the backward pass needs the same row histogram the forward pass has just
 * counted).  KEEP_HIST on lutb_product_forward: lay the workspace out as lutb_product_backward does and leave the
 * histogram in it.  REUSE_HIST on lutb_product_backward: the caller vouches that `workspace` is the one such a forward
 * call over the SAME x1, x2, positional embeddings and anchors used, untouched since: the pass skips its own counting.
 * Both only take effect when the histogram path runs and the whole batch goes through in one pass;
 * lutb_product_keeps_histogram(cfg, batch, S, n_inputs_1, n_inputs_2, variant, workspace, workspace_bytes) returns 1
 * exactly then (same variant, workspace pointer and size as the two calls; a workspace of
 * lutb_product_workspace(cfg, batch, S, 1) bytes qualifies whenever the histogram path is chosen).  Otherwise the
 * flags are ignored.
 */
#define LUTB_PRODUCT_KEEP_HIST 0x100
#define LUTB_PRODUCT_REUSE_HIST 0x200
int lutb_product_keeps_histogram(const lutb_layer_cfg *cfg, int64_t batch, int32_t seq_len, int32_t n_inputs_1,
                                 int32_t n_inputs_2, int variant, void *workspace, size_t workspace_bytes);
size_t lutb_product_workspace(const lutb_layer_cfg *cfg, int64_t batch, int32_t seq_len, int backward);

/*
 * Product-mode sequence layer, backward.  Replaces LUTDataManager::backward_backprop_product
 * (spiky_cuda/lut/lut.cu:945-1028 -> LUTRuntimeContext::backward_backprop_product, lut_runtime.cu:1051-1463).
 * Indices are recomputed; dX1 / dX2 (may alias) and dPE are accumulated into; dW / external_lr as in
 * lutb_nonseq_fc_backward.
 */
int lutb_product_backward(const lutb_layer_cfg *cfg, int64_t batch, int32_t seq_len, float *weights, const float *x1,
                          const float *x2, int32_t n_inputs_1, int32_t n_inputs_2, const float *pos_embeddings,
                          const int32_t *anchors, const float *dY, float *dX1, float *dX2, float *dPE, float *dW,
                          double external_lr, int variant, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Concatenation-mode sequence layer, forward.  Replaces LUTDataManager::forward_step_concat
 * (spiky_cuda/lut/lut.cu:718-845 -> LUTRuntimeContext::forward_step_concat, lut_runtime.cu:399-593).
 * cfg->seq_len = S > 1, cfg->n_inputs = inputs per token.  Tables have 2^(2*Nc + pos_dim) rows; pair (i < j)
 * selects row (idx[b,j,t] << (Nc + pos_dim)) | (idx[b,i,t] << pos_dim) | pos_idx[j-i-1, t].
 *   x fp32 [batch * S * I]; pos_embeddings fp32 [(S-1) * Nt * pos_dim] or NULL; y fp32 [batch * S * O] accumulated
 *   idx int32 [batch * S * Nt] out; min_delta / min_k [batch * S * Nt] out (both NULL = eval)
 *   pos_idx int32 [(S-1) * Nt] out, pos_min_delta / pos_min_k likewise (training only); NULL when pos_dim == 0
 */
int lutb_concat_forward(const lutb_layer_cfg *cfg, int64_t batch, const float *weights, const float *x,
                        const int32_t *anchors, const float *pos_embeddings, float *y, int32_t *idx, float *min_delta,
                        int32_t *min_k, int32_t *pos_idx, float *pos_min_delta, int32_t *pos_min_k, void *stream);

/*
 * Concatenation-mode sequence layer, backward.  Replaces LUTDataManager::backward_backprop_concat
 * (spiky_cuda/lut/lut.cu:1090-1180 -> LUTRuntimeContext::backward_backprop_concat, lut_runtime.cu:595-850).
 * dX fp32 [batch * S * I] and dPE fp32 [(S-1) * Nt * pos_dim] are accumulated into; dW / external_lr as in
 * lutb_nonseq_fc_backward.
 */
int lutb_concat_backward(const lutb_layer_cfg *cfg, int64_t batch, float *weights, const float *dY,
                         const int32_t *anchors, const int32_t *idx, const float *min_delta, const int32_t *min_k,
                         const int32_t *pos_idx, const float *pos_min_delta, const int32_t *pos_min_k, float *dX,
                         float *dPE, float *dW, double external_lr, void *stream);

/*
 * The stages of the concatenation-mode layer as separate entry points, for ranks that shard the QUERY positions of a
 * long sequence (no counterpart in the single-process reference; the arithmetic is that of the kernels named):
 *   lutb_check_detectors       table index (and, with min_delta / min_k, the minimum-margin pair) of `rows` input rows:
 *                              check_detectors[_eval]_logic, lut_runtime_kernels_logic.proto:1050-1158.  A rank runs
 *                              it on its own tokens; the ranks then all-gather idx / min_delta / min_k.
 *   lutb_check_positional      positional indices, check_positional_embeddings[_eval]_logic, proto:1709-1805.
 *   lutb_concat_pairs_forward  fill_outputs_fully_connected_seq_logic (proto:1807-1904) for the queries
 *                              j in [j_begin, j_end) only: y[b, j, :] += sum over keys i < j of the pair's row.  idx
 *                              int32 [batch * S * Nt] holds ALL tokens; rows of y outside the range are untouched, so
 *                              the ranks' outputs are disjoint.
 *   lutb_concat_pairs_backward propagate_through_detectors_seq_fc_logic (proto:3629-3835) and
 *                              gather_w_gradients_seq_fc_cpu_logic (proto:3944-4044) for the pairs whose query lies in
 *                              [j_begin, j_end): dX (all S tokens: keys of other ranks' tokens receive gradient too),
 *                              dPE and dW are PARTIAL sums that the ranks add up.  fp32 accumulators only.
 * Running the two pair stages over [0, S) is lutb_concat_forward / lutb_concat_backward without their index stage.
 */
int lutb_check_detectors(const lutb_layer_cfg *cfg, int64_t rows, const float *x, const int32_t *anchors, int32_t *idx,
                         float *min_delta, int32_t *min_k, void *stream);
int lutb_check_positional(const lutb_layer_cfg *cfg, const float *pos_embeddings, int32_t *pos_idx, float *pos_min_delta,
                          int32_t *pos_min_k, void *stream);
int lutb_concat_pairs_forward(const lutb_layer_cfg *cfg, int64_t batch, const float *weights, const int32_t *idx,
                              const int32_t *pos_idx, float *y, int32_t j_begin, int32_t j_end, void *stream);
int lutb_concat_pairs_backward(const lutb_layer_cfg *cfg, int64_t batch, float *weights, const float *dY,
                               const int32_t *anchors, const int32_t *idx, const float *min_delta, const int32_t *min_k,
                               const int32_t *pos_idx, const float *pos_min_delta, const int32_t *pos_min_k, float *dX,
                               float *dPE, float *dW, double external_lr, int32_t j_begin, int32_t j_end, void *stream);

/*
 * Concatenation-mode sequence layer with sparse lookup -> output connectivity (the reference builds it with
 * Conv2DLUTLayer(sequence_length > 1, lut_receptive_field_shape = ...)).  Replace the sparse branches of
 * LUTDataManager::forward_step_concat / backward_backprop_concat: fill_outputs_sparse_seq_logic
 * (lut_runtime_kernels_logic.proto:1906-2013), propagate_through_detectors_seq_sparse_logic (:3371-3627) and
 * gather_w_gradients_seq_sparse_logic (:3837-3942).  Arguments as lutb_concat_forward / lutb_concat_backward plus
 * the connectivity; the index holds 2^(2*Nc + pos_dim) rows per detector and weights is fp32 [sparse->n_weights].
 * (Product-mode layers with sparse connectivity are not provided: the reference's layer classes cannot construct
 * one, so no caller reaches that branch and nothing pins its results.)
 */
int lutb_concat_sparse_forward(const lutb_layer_cfg *cfg, const lutb_sparse_index *sparse, int64_t batch,
                               const float *weights, const float *x, const int32_t *anchors, const float *pos_embeddings,
                               float *y, int32_t *idx, float *min_delta, int32_t *min_k, int32_t *pos_idx,
                               float *pos_min_delta, int32_t *pos_min_k, void *stream);
int lutb_concat_sparse_backward(const lutb_layer_cfg *cfg, const lutb_sparse_index *sparse, int64_t batch, float *weights,
                                const float *dY, const int32_t *anchors, const int32_t *idx, const float *min_delta,
                                const int32_t *min_k, const int32_t *pos_idx, const float *pos_min_delta,
                                const int32_t *pos_min_k, float *dX, float *dPE, float *dW, double external_lr,
                                void *stream);

/*
 * Forward-only inference with int8 tables (non-sequence, fully connected).  No counterpart in the reference,
 * which has no quantised tables: the result is DEFINED as the reference's int32 fixed-point forward
 * (LUTDataManagerI::forward_step, spiky_cuda/lut/lut.cu:629-716 with INTEGERS_INSTEAD_OF_FLOATS) run on the
 * de-quantised table f32(scales[t] * q_tables[t][row][o]).
 *   q_tables int8 [Nt * 2^Nc * O] (O a multiple of 4), scales fp32 [Nt], x fp32 [batch * I]
 *   acc int32 [batch * O]: fixed-point accumulators, ADDED to (zero them first); idx int32 [batch * Nt] out
 * The accumulators of detector shards (each a multiple of cfg->backward_group detectors) add up exactly, on one
 * GPU or across GPUs; lutb_fixed_to_float then converts in place: y = f32(double(acc) * 2^-20-ish / int_rescaler)
 * (convert_integers_to_floats_logic, lut_runtime_kernels_logic.proto:200-213).
 * dequant selects what a table entry is: LUTB_INT8_DEQUANT_F32 the fp32 number f32(scale * q) (the table the
 * reference would be handed; slower: two conversions per entry), LUTB_INT8_DEQUANT_EXACT the exact real
 * scale * q (evaluated in fp64, where the 24 x 8 bit product is exact).  The two differ by at most the fp32
 * rounding of one entry (6e-8 relative) before the block truncation.
 */
#define LUTB_INT8_DEQUANT_F32 0
#define LUTB_INT8_DEQUANT_EXACT 1
int lutb_infer_int8_accumulate(const lutb_layer_cfg *cfg, int64_t batch, const int8_t *q_tables, const float *scales,
                               const float *x, const int32_t *anchors, int32_t *acc, int32_t *idx, int dequant,
                               void *stream);
int lutb_fixed_to_float(float *buffer, int64_t n, double int_rescaler, void *stream);

/*
 * Compaction of a dense 32-bit array (fp32 or int32 bit patterns) into sorted (index, value) lists: what the Sparse
 * gradient policy runs on the dense table gradient.  Replaces DenseToSparseConverterNative::count_nonzero and
 * ::dense_to_sparse_32 (spiky_cuda/torch_utils/torch_utils.cu:212-322 and :29-210; kernels densify_logic,
 * count_nonzero_logic, densify_new_logic in spiky_cuda/torch_utils/torch_utils_kernels_logic.proto:1-324).  Differences: positions come from a prefix sum, so the lists are in index
 * order and deterministic (the reference's order depends on scheduling); the scratch is a caller workspace of
 * lutb_dense_to_sparse_workspace(n) bytes instead of a counter tensor.
 *   source 32-bit words [n] (device); count_out int64 (device): number of non-zero words
 *   indices int64 [capacity], values 32-bit [capacity]: the first min(count, capacity) entries are written
 *   erase_input != 0: the source is zeroed (the shared gradient buffer is handed to the next layer clean)
 */
size_t lutb_dense_to_sparse_workspace(int64_t n);
int lutb_count_nonzero_32(const void *source, int64_t n, int64_t *count_out, void *workspace, size_t workspace_bytes,
                          void *stream);
int lutb_dense_to_sparse_32(void *source, int64_t n, int64_t *indices, void *values, int64_t capacity,
                            int64_t *count_out, int erase_input, void *workspace, size_t workspace_bytes, void *stream);

/*
 * fp32 GEMM on the sm_100a tensor cores with fp32-class accuracy (no reference counterpart; the reference has no
 * dense contraction): C [m x n] row-major = alpha * op(A) . op(B) + beta * C.  Default route: every operand is written
 * once as hi (x rounded to TF32) and lo = x - hi, and hi.hi + hi.lo + lo.hi is formed by TF32 GEMMs on concatenated
 * copies (tcgen05.mma, fp32 accumulators in tensor memory, operands staged by TMA); with
 * LUTB_GEMM_FAST_FP32 or'ed into `kind` a single GEMM splits the operands into BF16 terms inside its mainloop
 * instead (no scratch copies, about half the speed).  Either way results agree with an fp32 FMA contraction to about
 * 1e-6 relative.  The long-sequence (histogram) path of the product-mode layer runs its three contractions through the
 * default route.
 *   kind  LUTB_GEMM_A_ROWS_B_ROWS_OF_N: A [m x k] row-major, B stored as [n x k] row-major (C = A . B^T)
 *         LUTB_GEMM_A_ROWS_B_ROWS_OF_K: A [m x k] row-major, B stored as [k x n] row-major (C = A . B)
 *         LUTB_GEMM_A_COLS_B_ROWS_OF_K: A stored as [k x m] row-major, B as [k x n] row-major (C = A^T . B)
 * Pointers 16-byte aligned, leading dimensions and row lengths multiples of 4; workspace of
 * lutb_fp32_gemm_workspace(m, n, k) bytes (it holds the hi / lo copies).
 * lutb_fp32_gemm_available() is 0 when the library was built without a CUTLASS header tree (the call then fails with
 * LUTB_ERR_MODE and the histogram path keeps its fp32 FMA contractions).
 */
#define LUTB_GEMM_A_ROWS_B_ROWS_OF_N 0
#define LUTB_GEMM_A_ROWS_B_ROWS_OF_K 1
#define LUTB_GEMM_A_COLS_B_ROWS_OF_K 2
#define LUTB_GEMM_FAST_FP32 16
int lutb_fp32_gemm_available(void);
size_t lutb_fp32_gemm_workspace(int32_t m, int32_t n, int32_t k);
int lutb_fp32_gemm(int kind, int32_t m, int32_t n, int32_t k, const float *a, int64_t lda, const float *b, int64_t ldb,
                   float *c, int64_t ldc, float alpha, float beta, void *workspace, size_t workspace_bytes, void *stream);

/*
 * Data-parallel SGD over peer memory (no reference counterpart: the reference trains on one device).
 * lutb_peer_alloc allocates device memory other processes of the node can map and writes its 64-byte handle;
 * lutb_peer_open maps a buffer another process allocated (the handle travels by any host channel) and enables peer
 * access to its device; lutb_peer_close / lutb_peer_free undo them.  A handle cannot be opened in the process that
 * made it: that process uses the pointer it got from lutb_peer_alloc.
 * lutb_peer_sgd_update: rank `rank` of `n_ranks` owns floats [begin, end) of a table set.  grads[r] / weights[r] are
 * rank r's dense gradient and tables (own pointers or mapped ones, 16-byte aligned, same layout on every rank).  One
 * kernel computes, for every owned element e,  w = weights[rank][e] - scale * (grads[0][e] + ... + grads[n-1][e])
 * (fp32, summed in rank order, multiply and subtract rounded separately) and stores w into weights[r][e] of every
 * rank.  The kernel waits on nothing: the caller makes sure every rank's gradient is complete before any rank
 * launches it and that nobody reads the tables or rewrites the gradients before every rank's kernel has finished.
 * lutb_peer_broadcast: copies `bytes` from `src` (this rank's memory) to dst[r] + dst_offset of every listed buffer
 * (own pointers or mapped ones) with plain stores; 16-byte aligned offsets copy fastest.  Same ordering contract as
 * lutb_peer_sgd_update.
 * lutb_peer_copy: one asynchronous device-to-device copy on the stream (either side may be a mapped buffer of another
 * rank: the copy then runs on a copy engine over NVLink, without SMs).
 * lutb_peer_barrier: a barrier over the ranks on the stream, without the host: flags[r] is rank r's array of
 * 2 * LUTB_MAX_PEER_RANKS 64-bit words in shareable memory (zero before the first use: one flag per rank, then the
 * rank's own barrier count); every rank calls it with the same epoch, 1, 2, 3, ..., or with epoch 0: the kernel then
 * counts the barriers itself in device memory, and the launch, having no changing argument, can be part of a CUDA
 * graph that is replayed.
 * A kernel of one warp stores the epoch into this rank's slot of every rank's array (release at system scope, so what
 * earlier kernels of the stream wrote is visible to the ranks that see the flag) and waits until every slot of its own
 * array holds it.  The wait is bounded (about two seconds); one that runs out is counted by lutb_device_wait_errors and
 * the kernel returns.  Every rank must be running on its own GPU.
 */
#define LUTB_PEER_HANDLE_BYTES 64
#define LUTB_MAX_PEER_RANKS 16
int lutb_peer_alloc(size_t bytes, void **ptr_out, unsigned char *handle_out);
int lutb_peer_free(void *ptr);
int lutb_peer_open(const unsigned char *handle, void **ptr_out);
int lutb_peer_close(void *ptr);
int lutb_peer_broadcast(int32_t n_ranks, void *const *dst, int64_t dst_offset, const void *src, int64_t bytes,
                        void *stream);
int lutb_peer_copy(void *dst, const void *src, size_t bytes, void *stream);
int lutb_peer_barrier(int32_t n_ranks, int32_t rank, void *const *flags, uint64_t epoch, void *stream);
int lutb_peer_sgd_update(int32_t n_ranks, int32_t rank, const float *const *grads, float *const *weights,
                         int64_t begin, int64_t end, float scale, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SPIKY_B200_H */
