// Non-sequence LUT layer with sparse lookup -> output connectivity (projection / convolution layers).
// Each table row holds one weight per target of its detector; all rows of a detector share the target
// list, so the layer is a set of small fully connected tables whose outputs are scattered to shared
// output cells.
#include "lutb_common.cuh"
#include "nonseq_fc.cuh"

namespace lutb {

struct SparseView {
    const int64_t *det_wbase;
    const int32_t *det_stride;
    const int32_t *det_count;
    const int32_t *det_sstart;
    const int32_t *syn_det;
    const int32_t *syn_target;
    int64_t n_syn;
    int32_t group;
    int32_t group_shift;  // log2(group) when group is a power of two, else -1
};

__device__ __forceinline__ int hole_offset(int p, const SparseView &sp) {
    // two unused slots in front of every group of `group` synapses (the first pair lies before the row base)
    return 2 * (sp.group_shift >= 0 ? (p >> sp.group_shift) : (p / sp.group));
}

// --------------------------------------------------------------------------------------------
// Forward: y[b, target(t, p)] += W[slot(t, idx[b, t], p)] over all (detector, synapse) pairs
// (reference: fill_outputs_non_seq_sparse_logic + fire_single_synapse_group, proto:1160-1212, 215-313).
// A block owns one sample and a slice of the flattened pair list; the sample's index row and the
// output accumulators live in shared memory; consecutive threads read consecutive weights of a row.
// --------------------------------------------------------------------------------------------
template <bool INT_MODE>
__global__ void __launch_bounds__(256) sparse_forward_kernel(SparseView sp, const float *__restrict__ W,
                                                            const int32_t *__restrict__ idx, float *__restrict__ y,
                                                            int n_outputs, int n_detectors, int slices,
                                                            double fixed_scale) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *ys = reinterpret_cast<float *>(smem_raw);
    int32_t *yi = reinterpret_cast<int32_t *>(smem_raw);
    int32_t *idx_s = reinterpret_cast<int32_t *>(smem_raw) + n_outputs;
    const int64_t b = blockIdx.x;
    const int slice = blockIdx.y;
    const int64_t per = (sp.n_syn + slices - 1) / slices;
    const int64_t s0 = slice * per, s1 = min(sp.n_syn, s0 + per);
    for (int o = threadIdx.x; o < n_outputs; o += blockDim.x) yi[o] = 0;
    const int32_t *idx_b = idx + b * n_detectors;
    for (int t = threadIdx.x; t < n_detectors; t += blockDim.x) idx_s[t] = __ldg(idx_b + t);
    __syncthreads();
    for (int64_t s = s0 + threadIdx.x; s < s1; s += blockDim.x) {
        const int t = __ldg(sp.syn_det + s);
        const int target = __ldg(sp.syn_target + s);
        const int p = (int)(s - __ldg(sp.det_sstart + t));
        const int64_t slot = __ldg(sp.det_wbase + t) + (int64_t)idx_s[t] * __ldg(sp.det_stride + t) + p + hole_offset(p, sp);
        const float w = __ldg(W + slot);
        if (INT_MODE) atomicAdd(yi + target, to_fixed((double)w, fixed_scale));
        else atomicAdd(ys + target, w);
    }
    __syncthreads();
    if (INT_MODE) {
        int32_t *yb = reinterpret_cast<int32_t *>(y) + b * n_outputs;
        for (int o = threadIdx.x; o < n_outputs; o += blockDim.x) {
            const int32_t v = yi[o];
            if (v != 0) {
                if (slices == 1) yb[o] += v;
                else atomicAdd(yb + o, v);
            }
        }
    } else {
        float *yb = y + b * n_outputs;
        for (int o = threadIdx.x; o < n_outputs; o += blockDim.x) {
            const float v = ys[o];
            if (slices == 1) yb[o] += v;
            else if (v != 0.f) atomicAdd(yb + o, v);
        }
    }
}

// --------------------------------------------------------------------------------------------
// Input gradient (reference: propagate_through_detectors_non_seq_sparse_logic, proto:1303-1419).
// fp32 mode: a lane group of LG lanes owns one (sample, detector); lanes cover the synapses, the
// dot product dY[target] * (W[row] - W[alt]) is accumulated in double and reduced with shuffles.
// --------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) sparse_input_grad_kernel(SparseView sp, const float *__restrict__ W,
                                                               const float *__restrict__ dY,
                                                               const int2 *__restrict__ anchors,
                                                               const int32_t *__restrict__ idx,
                                                               const float *__restrict__ min_delta,
                                                               const int32_t *__restrict__ min_k,
                                                               float *__restrict__ dX, int n_inputs, int n_outputs,
                                                               int n_detectors, int n_anchors, int lanes_per_det,
                                                               int slices) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *dys = reinterpret_cast<float *>(smem_raw);
    const int64_t b = blockIdx.x;
    const float *dy = dY + b * n_outputs;
    for (int o = threadIdx.x; o < n_outputs; o += blockDim.x) dys[o] = __ldg(dy + o);
    __syncthreads();
    const int LG = lanes_per_det;
    const int groups_per_block = blockDim.x / LG;
    const int g = threadIdx.x / LG;
    const int j = threadIdx.x - g * LG;
    const unsigned lane = threadIdx.x & 31;
    const unsigned group_mask = (LG == 32) ? 0xffffffffu : (((1u << LG) - 1u) << (lane & ~(unsigned)(LG - 1)));
    const int per = (n_detectors + slices - 1) / slices;
    const int t_begin = blockIdx.y * per, t_end = min(n_detectors, t_begin + per);
    float *dx = dX + b * n_inputs;
    const int64_t base = b * n_detectors;
    for (int t0 = t_begin; t0 < t_end; t0 += groups_per_block) {
        const int t = t0 + g;
        const bool valid = t < t_end;
        double acc = 0.0;
        int32_t k = 0;
        if (valid) {
            const int32_t li = __ldg(idx + base + t);
            k = __ldg(min_k + base + t);
            const int P = __ldg(sp.det_count + t);
            const int64_t wbase = __ldg(sp.det_wbase + t);
            const int stride = __ldg(sp.det_stride + t);
            const int32_t *tg = sp.syn_target + __ldg(sp.det_sstart + t);
            const float *row = W + wbase + (int64_t)li * stride;
            const float *alt = W + wbase + (int64_t)(li ^ (1 << k)) * stride;
            for (int p = j; p < P; p += LG) {
                const int q = p + hole_offset(p, sp);
                acc += (double)dys[__ldg(tg + p)] * ((double)__ldg(row + q) - (double)__ldg(alt + q));
            }
        }
        for (int off = 1; off < LG; off <<= 1) acc += __shfl_xor_sync(group_mask, acc, off);
        if (valid && j == 0) {
            const double du = surrogate_up(__ldg(min_delta + base + t)) * acc;
            if (fabs(du) > kEps) {
                const int2 a = __ldg(anchors + (size_t)t * n_anchors + k);
                atomicAdd(dx + a.x, (float)du);
                atomicAdd(dx + a.y, -(float)du);
            }
        }
    }
}

// Fixed-point variant: one thread per (sample, detector) walks the synapse groups in order; each group's
// du is truncated on its own (bit-exact with the reference), integer atomics make the order irrelevant.
__global__ void sparse_input_grad_fixed_kernel(SparseView sp, const float *__restrict__ W, const float *__restrict__ dY,
                                               const int2 *__restrict__ anchors, const int32_t *__restrict__ idx,
                                               const float *__restrict__ min_delta, const int32_t *__restrict__ min_k,
                                               float *__restrict__ dX, int64_t batch, int n_inputs, int n_outputs,
                                               int n_detectors, int n_anchors, double fixed_scale) {
    const int64_t total = batch * n_detectors;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / n_detectors;
        const int t = (int)(i - b * n_detectors);
        const int32_t li = idx[i];
        const int32_t k = min_k[i];
        const double up = surrogate_up(min_delta[i]);
        const int P = sp.det_count[t];
        const int64_t wbase = sp.det_wbase[t];
        const int stride = sp.det_stride[t];
        const int32_t *tg = sp.syn_target + sp.det_sstart[t];
        const float *row = W + wbase + (int64_t)li * stride;
        const float *alt = W + wbase + (int64_t)(li ^ (1 << k)) * stride;
        const float *dy = dY + b * n_outputs;
        const int2 a = __ldg(anchors + (size_t)t * n_anchors + k);
        int32_t *dx = reinterpret_cast<int32_t *>(dX) + b * n_inputs;
        for (int p0 = 0; p0 < P; p0 += sp.group) {
            const int p1 = min(p0 + sp.group, P);
            double ms = 0.0, as = 0.0;
            for (int p = p0; p < p1; p++) ms += (double)__ldg(row + p + hole_offset(p, sp)) * (double)__ldg(dy + tg[p]);
            for (int p = p0; p < p1; p++) as += (double)__ldg(alt + p + hole_offset(p, sp)) * (double)__ldg(dy + tg[p]);
            const double du = up * (ms - as);
            if (fabs(du) > kEps) {
                const int32_t d = to_fixed(du, fixed_scale);
                atomicAdd(dx + a.x, d);
                atomicAdd(dx + a.y, -d);
            }
        }
    }
}

// --------------------------------------------------------------------------------------------
// Table gradient: target[slot(t, idx[b, t], p)] += lr * dY[b, target(t, p)] for |dY| > EPS
// (reference: gather_w_gradients_non_seq_sparse_logic, proto:1501-1545, helper :584-714).
// Same flattened pair list as the forward; consecutive threads update consecutive slots of a row.
// --------------------------------------------------------------------------------------------
template <bool INT_MODE>
__global__ void __launch_bounds__(256) sparse_weight_grad_kernel(SparseView sp, const float *__restrict__ dY,
                                                                const int32_t *__restrict__ idx,
                                                                float *__restrict__ target_arr, int n_outputs,
                                                                int n_detectors, int slices, double lr,
                                                                double fixed_scale) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float *dys = reinterpret_cast<float *>(smem_raw);
    int32_t *idx_s = reinterpret_cast<int32_t *>(smem_raw) + n_outputs;
    const int64_t b = blockIdx.x;
    const int64_t per = (sp.n_syn + slices - 1) / slices;
    const int64_t s0 = blockIdx.y * per, s1 = min(sp.n_syn, s0 + per);
    const float *dy = dY + b * n_outputs;
    for (int o = threadIdx.x; o < n_outputs; o += blockDim.x) dys[o] = __ldg(dy + o);
    const int32_t *idx_b = idx + b * n_detectors;
    for (int t = threadIdx.x; t < n_detectors; t += blockDim.x) idx_s[t] = __ldg(idx_b + t);
    __syncthreads();
    for (int64_t s = s0 + threadIdx.x; s < s1; s += blockDim.x) {
        const int t = __ldg(sp.syn_det + s);
        const double g = (double)dys[__ldg(sp.syn_target + s)];
        if (fabs(g) > kEps) {
            const int p = (int)(s - __ldg(sp.det_sstart + t));
            const int64_t slot = __ldg(sp.det_wbase + t) + (int64_t)idx_s[t] * __ldg(sp.det_stride + t) + p + hole_offset(p, sp);
            if (INT_MODE) atomicAdd(reinterpret_cast<int32_t *>(target_arr) + slot, to_fixed(g * lr, fixed_scale));
            else atomicAdd(target_arr + slot, (float)(g * lr));
        }
    }
}

static SparseView make_view(const lutb_sparse_index *sp) {
    SparseView v;
    v.det_wbase = sp->det_wbase; v.det_stride = sp->det_stride; v.det_count = sp->det_count;
    v.det_sstart = sp->det_sstart; v.syn_det = sp->syn_det; v.syn_target = sp->syn_target;
    v.n_syn = sp->n_syn_per_sample; v.group = sp->group_size;
    v.group_shift = -1;
    for (int s = 0; s < 31; s++) if ((1 << s) == sp->group_size) v.group_shift = s;
    return v;
}

static int validate_sparse(const lutb_sparse_index *sp) {
    LUTB_REQUIRE(sp != nullptr, LUTB_ERR_NULL, "sparse index is NULL");
    LUTB_REQUIRE(sp->det_wbase && sp->det_stride && sp->det_count && sp->det_sstart && sp->syn_det && sp->syn_target,
                 LUTB_ERR_NULL, "a sparse index array is NULL");
    LUTB_REQUIRE(sp->group_size > 0 && sp->n_syn_per_sample > 0 && sp->n_weights > 0 && sp->max_count > 0,
                 LUTB_ERR_SHAPE, "empty sparse index");
    return LUTB_OK;
}

static int pick_slices(int64_t batch, int sm, int64_t work_items, int min_items) {
    // enough blocks for ~4 per SM, but never slices with fewer than `min_items` work items
    int64_t want = ((int64_t)sm * 4 + batch - 1) / batch;
    int64_t cap = max((int64_t)1, work_items / min_items);
    return (int)max((int64_t)1, min(min(want, cap), (int64_t)64));
}

}  // namespace lutb

using namespace lutb;

extern "C" int lutb_nonseq_sparse_forward(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                          const float *weights, const float *x, const int32_t *anchors, float *y,
                                          int32_t *idx, float *min_delta, int32_t *min_k, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    rc = validate_sparse(sp);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->seq_len == 1, LUTB_ERR_MODE, "forward_step should only be called when sequence_length == 1");
    LUTB_REQUIRE(batch > 0 && batch <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "batch_size == 0 or too large");
    LUTB_REQUIRE(weights && x && anchors && y && idx, LUTB_ERR_NULL, "a required tensor pointer is NULL");
    LUTB_REQUIRE((min_delta == nullptr) == (min_k == nullptr), LUTB_ERR_MODE,
                 "min_anchor_deltas and min_anchor_delta_indices must be given together");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    rc = launch_check_detectors(x, batch, cfg->n_inputs, anchors, cfg->n_detectors, cfg->n_anchors, cfg->cmp_eps, idx,
                                min_delta, min_k, st);
    if (rc) return rc;
    const size_t smem = (size_t)(cfg->n_outputs + cfg->n_detectors) * 4;
    LUTB_REQUIRE(smem <= (size_t)kMaxSmemPerBlock - 1024, LUTB_ERR_SHAPE,
                 "n_outputs + n_detectors too large for the sparse forward kernel");
    const int slices = pick_slices(batch, device_info().sm_count, sp->n_syn_per_sample, 4096);
    SparseView v = make_view(sp);
    dim3 grid((unsigned)batch, (unsigned)slices);
    {
        KernelScope scope(K_SPARSE_FORWARD, st);
        if (cfg->int_mode) {
            if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(sparse_forward_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            sparse_forward_kernel<true><<<grid, 256, smem, st>>>(v, weights, idx, y, cfg->n_outputs, cfg->n_detectors, slices, cfg->int_rescaler);
        } else {
            if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(sparse_forward_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            sparse_forward_kernel<false><<<grid, 256, smem, st>>>(v, weights, idx, y, cfg->n_outputs, cfg->n_detectors, slices, cfg->int_rescaler);
        }
    }
    LUTB_LAUNCH_CHECK();
    if (cfg->int_mode) return launch_fixed_to_float(y, batch * (int64_t)cfg->n_outputs, cfg->int_rescaler, st);
    return LUTB_OK;
}

extern "C" int lutb_nonseq_sparse_backward(const lutb_layer_cfg *cfg, const lutb_sparse_index *sp, int64_t batch,
                                           float *weights, const float *dY, const int32_t *anchors,
                                           const int32_t *idx, const float *min_delta, const int32_t *min_k,
                                           float *dX, float *dW, double external_lr, void *stream) {
    int rc = validate_cfg(cfg);
    if (rc) return rc;
    rc = validate_sparse(sp);
    if (rc) return rc;
    LUTB_REQUIRE(cfg->seq_len == 1, LUTB_ERR_MODE, "backward_backprop should only be called when sequence_length == 1");
    LUTB_REQUIRE(batch > 0 && batch <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "batch_size == 0 or too large");
    LUTB_REQUIRE(weights && dY && anchors && idx && min_delta && min_k && dX, LUTB_ERR_NULL,
                 "a required tensor pointer is NULL");
    LUTB_REQUIRE(!(external_lr >= 0.0 && dW != nullptr), LUTB_ERR_MODE,
                 "in internal weight gradients mode w_weights_gradients should be nullptr");
    LUTB_REQUIRE(!(external_lr < 0.0 && dW == nullptr), LUTB_ERR_NULL, "w_weights_gradients is NULL");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int sm = device_info().sm_count;
    SparseView v = make_view(sp);
    const int O = cfg->n_outputs, Nt = cfg->n_detectors;
    {
        KernelScope scope(K_SPARSE_INPUT_GRAD, st);
        if (cfg->int_mode) {
            const int64_t total = batch * Nt;
            const int64_t blocks = min((total + 127) / 128, (int64_t)sm * 64);
            sparse_input_grad_fixed_kernel<<<(unsigned)blocks, 128, 0, st>>>(
                v, weights, dY, reinterpret_cast<const int2 *>(anchors), idx, min_delta, min_k, dX, batch,
                cfg->n_inputs, O, Nt, cfg->n_anchors, cfg->int_rescaler);
        } else {
            int lanes = 1;
            while (lanes < 32 && lanes < sp->max_count) lanes <<= 1;
            const size_t smem = (size_t)O * 4;
            LUTB_REQUIRE(smem <= (size_t)kMaxSmemPerBlock - 1024, LUTB_ERR_SHAPE, "n_outputs too large for the sparse backward kernel");
            if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(sparse_input_grad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            const int slices = pick_slices(batch, sm, Nt, 256);
            dim3 grid((unsigned)batch, (unsigned)slices);
            sparse_input_grad_kernel<<<grid, 256, smem, st>>>(v, weights, dY, reinterpret_cast<const int2 *>(anchors), idx,
                                                             min_delta, min_k, dX, cfg->n_inputs, O, Nt, cfg->n_anchors,
                                                             lanes, slices);
        }
    }
    LUTB_LAUNCH_CHECK();
    double lr = cfg->lr_meta;
    if (external_lr >= 0.0) lr *= -(double)(float)external_lr;
    float *target = external_lr >= 0.0 ? weights : dW;
    {
        const size_t smem = (size_t)(O + Nt) * 4;
        LUTB_REQUIRE(smem <= (size_t)kMaxSmemPerBlock - 1024, LUTB_ERR_SHAPE,
                     "n_outputs + n_detectors too large for the sparse table-gradient kernel");
        const int slices = pick_slices(batch, sm, sp->n_syn_per_sample, 4096);
        dim3 grid((unsigned)batch, (unsigned)slices);
        KernelScope scope(K_SPARSE_WEIGHT_GRAD, st);
        if (cfg->int_mode) {
            if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(sparse_weight_grad_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            sparse_weight_grad_kernel<true><<<grid, 256, smem, st>>>(v, dY, idx, target, O, Nt, slices, lr, cfg->int_rescaler);
        } else {
            if (smem > 48 * 1024) LUTB_CUDA(cudaFuncSetAttribute(sparse_weight_grad_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            sparse_weight_grad_kernel<false><<<grid, 256, smem, st>>>(v, dY, idx, target, O, Nt, slices, lr, cfg->int_rescaler);
        }
    }
    LUTB_LAUNCH_CHECK();
    if (cfg->int_mode) {
        rc = launch_fixed_to_float(dX, batch * (int64_t)cfg->n_inputs, cfg->int_rescaler, st);
        if (rc) return rc;
        if (dW) rc = launch_fixed_to_float(dW, sp->n_weights, cfg->int_rescaler, st);
    }
    return rc;
}
