// Launchers shared between the non-sequence and the sequence (concatenation) entry points.
#pragma once
#include "lutb_common.cuh"

namespace lutb {

// Anchor comparison + bit packing for `rows` input rows of `n_inputs` floats.
// min_delta / min_k NULL selects the evaluation variant.
int launch_check_detectors(const float *x, int64_t rows, int n_inputs, const int32_t *anchors, int n_detectors,
                           int n_anchors, float cmp_eps, int32_t *idx, float *min_delta, int32_t *min_k,
                           cudaStream_t stream);

// y[b, :] += sum_t W[t, idx[b, t], :] (int_mode: y holds int32 fixed-point cells, not yet converted).
int launch_fc_gather_forward(const float *W, const int32_t *idx, float *y, int64_t batch, int n_outputs,
                             int n_detectors, int table_rows, int det_block, bool int_mode, double fixed_scale,
                             cudaStream_t stream);

}  // namespace lutb
