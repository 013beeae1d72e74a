// Table-ownership ("staged") kernels of the sparse non-sequence layer: forward and input gradient.
// See sparse_staged.cu for the design.
#pragma once

#include "lutb_common.cuh"

namespace lutb {

// True when the staged kernels can run this layer: fp32 accumulators, rows of at most 32 synapses, every detector
// table 16-byte aligned and small enough that at least three of them fit the shared-memory ring.
bool sparse_staged_possible(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, const float *weights);

// The library's choice between the gather kernels (one warp per (chunk, few samples), rows fetched through L2) and
// the staged kernels (whole tables streamed through shared memory once per 512 samples): staged pays when most rows
// of a table are selected by some sample of the batch anyway.  pass 0 = forward, 1 = input gradient.
bool sparse_staged_preferred(int pass, const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch);

// y[b, target(p)] += sum over detectors of W[row(t, idx[b, t]) + p]      (fill_outputs_non_seq_sparse)
int launch_sparse_forward_staged(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                 const float *weights, const int32_t *idx, float *y, cudaStream_t stream);

// dX[b, anchor(t, min_k)] +-= up(min_delta) * sum_p dY[b, target(p)] * (W[row + p] - W[alt + p])
// (propagate_through_detectors_non_seq_sparse)
int launch_sparse_input_grad_staged(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                    const float *weights, const float *dY, const int32_t *anchors, const int32_t *idx,
                                    const float *min_delta, const int32_t *min_k, float *dX, cudaStream_t stream);

}  // namespace lutb
