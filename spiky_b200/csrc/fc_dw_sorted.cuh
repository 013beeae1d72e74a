// Sorted (deterministic) table-gradient variant of the non-sequence fully connected layer.
#pragma once
#include "lutb_common.cuh"

namespace lutb {

// bytes of int32 scratch: per-(detector, row, 1024-sample block) counters + the sorted sample lists
size_t fc_dw_sorted_workspace(int64_t batch, int n_detectors, int table_rows);

// target[t, idx[b, t], :] += lr * dY[b, :] (|dY| > EPS), samples added in ascending order per cell.
// `workspace` must hold fc_dw_sorted_workspace() bytes.
int launch_fc_dw_sorted(const float *dY, const int32_t *idx, float *target, int64_t batch, int n_outputs,
                        int n_detectors, int table_rows, double lr, void *workspace, cudaStream_t stream,
                        bool clear_with_memset = true);

// The table gradient as a list of touched rows: row_ids[k] = detector * table_rows + row in ascending order,
// values[k * n_outputs + o] the row's sums (ascending sample order per cell), *count_out the number of touched rows
// (rows beyond `capacity` are counted but not written).  `workspace` must hold fc_dw_rows_workspace() bytes.
size_t fc_dw_rows_workspace(int64_t batch, int n_detectors, int table_rows);
int launch_fc_dw_rows(const float *dY, const int32_t *idx, int64_t batch, int n_outputs, int n_detectors, int table_rows,
                      double lr, int64_t *row_ids, float *values, int64_t capacity, int64_t *count_out, void *workspace,
                      cudaStream_t stream);

// Device address (on the current device) of the library's built-in scratch array of
// LUTB_STATIC_SCRATCH_BYTES bytes; resolved once per device on first use.
int static_scratch(void **ptr);

}  // namespace lutb
