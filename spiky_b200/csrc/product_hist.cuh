// Histogram formulation of the product-mode sequence layer for long sequences (fp32 accumulators).
//
// For a query row (b, j) and detector t the S*(S-1)/2-pair sums of the layer only depend on how often each
// table row is selected: with H[t][(b,j)][r] = #{i < j : index(i, j, t) = r}
//     forward        y[(b,j), :]   += sum_t H_t[(b,j), :] . W_t                 (rows x T) . (T x O)
//     table gradient dW_t          += lr * H_t^T . dY                            (T x rows) . (rows x O)
//     input gradient g(i,j,t)       = Q_t[(b,j), idx] - Q_t[(b,j), alt],  Q_t = dY . W_t^T   (rows x O) . (O x T)
// so the row gathers and scatter-adds of the direct kernels (one table row per pair through L2) become dense
// contractions: fp32-accurate GEMMs on the tensor cores (fp32_gemm_sm100.cuh; the counters are then kept as fp32 in
// the layout [row][detector][T], so that each of the three sums is ONE GEMM over all detectors), or, without them,
// register-tiled fp32 FMA contractions whose table traffic is amortised over 128 query rows.  Worth it once a query
// has about as many keys as the table has rows.
#pragma once

#include "lutb_common.cuh"

namespace lutb {

struct ProductCall {
    const lutb_layer_cfg *cfg;
    int64_t batch;
    int S, e1, e2;
    const float *x1, *x2, *pe;
    const int32_t *anchors;
};

// Whether the shapes and alignments of a call allow the histogram kernels at all.
bool product_hist_supported(const ProductCall &c, const void *weights, const void *io_rows, const void *dW);
// Workspace bytes that let `batch` sequences through in one pass (the batch is processed in passes of as many whole
// sequences as the workspace holds).
size_t product_hist_workspace_bytes(const lutb_layer_cfg *cfg, int64_t batch, int S, bool backward);

// allow_tc: run the contractions on the tensor cores (fp32_gemm_sm100.cuh) when the library has them and the workspace
// holds at least one sequence in their operand layout; otherwise, and when false, the fp32 FMA contraction runs.
// keep: leave the row histogram in the workspace where launch_product_hist_backward(..., reuse = true) finds it
// (product_hist_keeps tells whether a workspace of that size allows it: the whole batch must be one pass).
bool product_hist_keeps(const ProductCall &c, bool allow_tc, void *workspace, size_t workspace_bytes);
int launch_product_hist_forward(const ProductCall &c, const float *weights, float *y, bool allow_tc, void *workspace,
                                size_t workspace_bytes, cudaStream_t stream, bool keep = false);
// target: dW (external gradients) or the tables themselves (in-place SGD: all input gradients first).
int launch_product_hist_backward(const ProductCall &c, const float *weights, const float *dY, float *dX1, float *dX2,
                                 float *dPE, float *target, double lr, bool in_place, bool allow_tc, void *workspace,
                                 size_t workspace_bytes, cudaStream_t stream, bool reuse = false);

}  // namespace lutb
