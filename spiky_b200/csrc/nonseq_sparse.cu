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
    const int32_t *syn_target;
    const int4 *chunks;   // (first detector, detector count <= 32, target list offset, synapses per row)
    int64_t n_chunks;
    int32_t group;
    int32_t group_shift;  // log2(group) when group is a power of two, else -1
};

__device__ __forceinline__ int hole_offset(int p, const SparseView &sp) {
    // two unused slots in front of every group of `group` synapses (the first pair lies before the row base)
    return 2 * (sp.group_shift >= 0 ? (p >> sp.group_shift) : (p / sp.group));
}

// All three training kernels give one warp to a (sample, chunk) pair.  A chunk is a run of up to 32
// consecutive detectors that share one target list (the detectors of one group).  Lane L first loads
// the table index of detector L of the chunk (one coalesced read) and turns it into the offset of the
// selected row relative to the chunk's first table; the offsets are then broadcast with shuffles while
// the lanes cover the synapses of a row, so that every row read or update is one contiguous segment.
// When rows are short the warp splits into NG = 32 / LG lane groups that take detectors round-robin.
struct ChunkLane {
    int det0, ndet, toff, P;
    int64_t wbase0;
    int32_t row_off;   // offset of this lane's detector's selected row from wbase0 (0 when lane >= ndet)
};

__device__ __forceinline__ ChunkLane load_chunk(const SparseView &sp, const int32_t *__restrict__ idx_b, int64_t c,
                                                int lane, int32_t *li_out) {
    const int4 ci = __ldg(sp.chunks + c);
    ChunkLane ch;
    ch.det0 = ci.x; ch.ndet = ci.y; ch.toff = ci.z; ch.P = ci.w;
    ch.wbase0 = __ldg(sp.det_wbase + ch.det0);
    ch.row_off = 0;
    int32_t li = 0;
    if (lane < ch.ndet) {
        const int t = ch.det0 + lane;
        li = __ldg(idx_b + t);
        ch.row_off = (int32_t)(__ldg(sp.det_wbase + t) - ch.wbase0) + li * __ldg(sp.det_stride + t);
    }
    if (li_out) *li_out = li;
    return ch;
}

// --------------------------------------------------------------------------------------------
// Forward: y[b, target(p)] += sum over the chunk's detectors of W[row(t, idx[b, t]) + p]
// (reference: fill_outputs_non_seq_sparse_logic + fire_single_synapse_group, proto:1160-1212, 215-313).
// The chunk's detectors are summed in registers, so the shared output cells see one reduction per
// (sample, chunk, target) instead of one per synapse.
// --------------------------------------------------------------------------------------------
template <bool INT_MODE>
__global__ void __launch_bounds__(256) sparse_forward_kernel(SparseView sp, const float *__restrict__ W,
                                                            const int32_t *__restrict__ idx, float *__restrict__ y,
                                                            int64_t batch, int n_outputs, int n_detectors,
                                                            double fixed_scale) {
    const int lane = threadIdx.x & 31;
    const int64_t work = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (work >= batch * sp.n_chunks) return;
    const int64_t b = work / sp.n_chunks;
    const int64_t c = work - b * sp.n_chunks;
    const ChunkLane ch = load_chunk(sp, idx + b * n_detectors, c, lane, nullptr);
    int LG = 32;
    while (LG > 4 && (LG >> 1) >= ch.P) LG >>= 1;
    const int NG = 32 / LG;
    const int g = lane / LG, j = lane - g * LG;
    const float *Wb = W + ch.wbase0;
    const int32_t *tg = sp.syn_target + ch.toff;
    for (int p0 = 0; p0 < ch.P; p0 += LG) {
        const int p = p0 + j;
        const bool valid = p < ch.P;
        const int q = p + hole_offset(p, sp);
        float acc = 0.f;
        int32_t iacc = 0;
#pragma unroll 4
        for (int d0 = 0; d0 < ch.ndet; d0 += NG) {
            const int d = d0 + g;
            const int32_t off = __shfl_sync(0xffffffffu, ch.row_off, d & 31);
            if (valid && d < ch.ndet) {
                const float w = __ldg(Wb + (int64_t)off + q);
                if (INT_MODE) iacc += to_fixed((double)w, fixed_scale);
                else acc += w;
            }
        }
        for (int m = LG; m < 32; m <<= 1) {
            if (INT_MODE) iacc += __shfl_xor_sync(0xffffffffu, iacc, m);
            else acc += __shfl_xor_sync(0xffffffffu, acc, m);
        }
        if (valid && g == 0) {
            const int target = __ldg(tg + p);
            if (INT_MODE) atomicAdd(reinterpret_cast<int32_t *>(y) + b * n_outputs + target, iacc);
            else atomicAdd(y + b * n_outputs + target, acc);
        }
    }
}

// --------------------------------------------------------------------------------------------
// Input gradient (reference: propagate_through_detectors_non_seq_sparse_logic, proto:1303-1419):
// per (sample, detector) g = sum_p dY[target(p)] * (W[row + p] - W[alt + p]), du = up(min_delta) * g.
// A lane group of LG lanes covers the synapses; every lane keeps one partial per detector it sees
// (LG of them), and a butterfly of LG - 1 shuffles transposes and reduces them so that each lane
// ends with the full sum of exactly one detector and performs that detector's two updates itself.
// Rows have at most 32 synapses here (longer rows use the generic kernel below); partial products are
// fp32 (<= 32 terms), the scaling by up() is done in double.
// --------------------------------------------------------------------------------------------
template <int LG>
__global__ void __launch_bounds__(256) sparse_input_grad_kernel(SparseView sp, const float *__restrict__ W,
                                                               const float *__restrict__ dY,
                                                               const int2 *__restrict__ anchors,
                                                               const int32_t *__restrict__ idx,
                                                               const float *__restrict__ min_delta,
                                                               const int32_t *__restrict__ min_k,
                                                               float *__restrict__ dX, int64_t batch, int n_inputs,
                                                               int n_outputs, int n_detectors, int n_anchors) {
    constexpr int NG = 32 / LG;
    const int lane = threadIdx.x & 31;
    const int64_t work = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (work >= batch * sp.n_chunks) return;
    const int64_t b = work / sp.n_chunks;
    const int64_t c = work - b * sp.n_chunks;
    int32_t li;
    const ChunkLane ch = load_chunk(sp, idx + b * n_detectors, c, lane, &li);
    // this lane's detector: alternative row (minimum-margin bit flipped), margin, flipped pair
    int32_t alt_off = 0, my_k = 0;
    float my_m = 0.f;
    if (lane < ch.ndet) {
        const int t = ch.det0 + lane;
        my_k = __ldg(min_k + b * n_detectors + t);
        my_m = __ldg(min_delta + b * n_detectors + t);
        alt_off = ch.row_off + ((li ^ (1 << my_k)) - li) * __ldg(sp.det_stride + t);
    }
    const int g = lane / LG, j = lane - g * LG;
    const bool valid = j < ch.P;
    const int q = j + hole_offset(j, sp);
    const float *Wb = W + ch.wbase0 + q;
    const float gp = valid ? __ldg(dY + b * n_outputs + __ldg(sp.syn_target + ch.toff + j)) : 0.f;
    float v[LG];
#pragma unroll
    for (int i = 0; i < LG; i++) {
        const int d = i * NG + g;
        const int32_t ro = __shfl_sync(0xffffffffu, ch.row_off, d);
        const int32_t ao = __shfl_sync(0xffffffffu, alt_off, d);
        // detectors beyond the chunk have ro == ao == 0: the difference below is exactly zero
        v[i] = valid ? gp * (__ldg(Wb + ro) - __ldg(Wb + ao)) : 0.f;
    }
    // transpose-reduce: after the stage with offset o, a lane keeps the half of the values whose
    // index bit matches its own lane bit, summed with the partner lane's copy
#pragma unroll
    for (int o = LG / 2; o >= 1; o >>= 1) {
        const bool upper = (j & o) != 0;
#pragma unroll
        for (int i = 0; i < o; i++) {
            const float send = upper ? v[i] : v[i + o];
            const float keep = upper ? v[i + o] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
    }
    // lane (g, j) now holds detector d = j * NG + g of the chunk
    const int d = j * NG + g;
    const int32_t k = __shfl_sync(0xffffffffu, my_k, d);
    const float m = __shfl_sync(0xffffffffu, my_m, d);
    if (d < ch.ndet) {
        const double du = surrogate_up(m) * (double)v[0];
        if (fabs(du) > kEps) {
            const int2 a = __ldg(anchors + (size_t)(ch.det0 + d) * n_anchors + k);
            float *dx = dX + b * n_inputs;
            atomicAdd(dx + a.x, (float)du);
            atomicAdd(dx + a.y, -(float)du);
        }
    }
}

// Generic fp32 input gradient for rows longer than 32 synapses: one warp per (sample, detector).
__global__ void __launch_bounds__(256) sparse_input_grad_long_kernel(SparseView sp, const float *__restrict__ W,
                                                                    const float *__restrict__ dY,
                                                                    const int2 *__restrict__ anchors,
                                                                    const int32_t *__restrict__ idx,
                                                                    const float *__restrict__ min_delta,
                                                                    const int32_t *__restrict__ min_k,
                                                                    float *__restrict__ dX, int64_t batch,
                                                                    int n_inputs, int n_outputs, int n_detectors,
                                                                    int n_anchors) {
    const int lane = threadIdx.x & 31;
    const int64_t work = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (work >= batch * n_detectors) return;
    const int64_t b = work / n_detectors;
    const int t = (int)(work - b * n_detectors);
    const int32_t li = __ldg(idx + work);
    const int32_t k = __ldg(min_k + work);
    const int P = __ldg(sp.det_count + t);
    const int64_t wbase = __ldg(sp.det_wbase + t);
    const int stride = __ldg(sp.det_stride + t);
    const int32_t *tg = sp.syn_target + __ldg(sp.det_sstart + t);
    const float *row = W + wbase + (int64_t)li * stride;
    const float *alt = W + wbase + (int64_t)(li ^ (1 << k)) * stride;
    const float *dy = dY + b * n_outputs;
    double acc = 0.0;
    for (int p = lane; p < P; p += 32) {
        const int q = p + hole_offset(p, sp);
        acc += (double)__ldg(dy + __ldg(tg + p)) * ((double)__ldg(row + q) - (double)__ldg(alt + q));
    }
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) {
        const double du = surrogate_up(__ldg(min_delta + work)) * acc;
        if (fabs(du) > kEps) {
            const int2 a = __ldg(anchors + (size_t)t * n_anchors + k);
            atomicAdd(dX + b * n_inputs + a.x, (float)du);
            atomicAdd(dX + b * n_inputs + a.y, -(float)du);
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
// Table gradient: target[row(t, idx[b, t]) + p] += lr * dY[b, target(p)] for |dY| > EPS
// (reference: gather_w_gradients_non_seq_sparse_logic, proto:1501-1545, helper :584-714).
// The value a lane adds is the same for all detectors of the chunk; every detector's row receives one
// contiguous run of reductions.
// --------------------------------------------------------------------------------------------
template <bool INT_MODE>
__global__ void __launch_bounds__(256) sparse_weight_grad_kernel(SparseView sp, const float *__restrict__ dY,
                                                                const int32_t *__restrict__ idx,
                                                                float *__restrict__ target_arr, int64_t batch,
                                                                int n_outputs, int n_detectors, double lr,
                                                                double fixed_scale) {
    const int lane = threadIdx.x & 31;
    const int64_t work = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (work >= batch * sp.n_chunks) return;
    const int64_t b = work / sp.n_chunks;
    const int64_t c = work - b * sp.n_chunks;
    const ChunkLane ch = load_chunk(sp, idx + b * n_detectors, c, lane, nullptr);
    int LG = 32;
    while (LG > 4 && (LG >> 1) >= ch.P) LG >>= 1;
    const int NG = 32 / LG;
    const int g = lane / LG, j = lane - g * LG;
    float *Tb = target_arr + ch.wbase0;
    const int32_t *tg = sp.syn_target + ch.toff;
    for (int p0 = 0; p0 < ch.P; p0 += LG) {
        const int p = p0 + j;
        const int q = p + hole_offset(p, sp);
        float val = 0.f;
        int32_t ival = 0;
        bool active = false;
        if (p < ch.P) {
            const double gd = (double)__ldg(dY + b * n_outputs + __ldg(tg + p));
            if (fabs(gd) > kEps) {
                active = true;
                if (INT_MODE) ival = to_fixed(gd * lr, fixed_scale);
                else val = (float)(gd * lr);
            }
        }
        for (int d0 = 0; d0 < ch.ndet; d0 += NG) {
            const int d = d0 + g;
            const int32_t off = __shfl_sync(0xffffffffu, ch.row_off, d & 31);
            if (active && d < ch.ndet) {
                if (INT_MODE) atomicAdd(reinterpret_cast<int32_t *>(Tb) + (int64_t)off + q, ival);
                else atomicAdd(Tb + (int64_t)off + q, val);
            }
        }
    }
}

static SparseView make_view(const lutb_sparse_index *sp) {
    SparseView v;
    v.det_wbase = sp->det_wbase; v.det_stride = sp->det_stride; v.det_count = sp->det_count;
    v.det_sstart = sp->det_sstart; v.syn_target = sp->syn_target;
    v.chunks = reinterpret_cast<const int4 *>(sp->chunk_info); v.n_chunks = sp->n_chunks; v.group = sp->group_size;
    v.group_shift = -1;
    for (int s = 0; s < 31; s++) if ((1 << s) == sp->group_size) v.group_shift = s;
    return v;
}

static int validate_sparse(const lutb_sparse_index *sp) {
    LUTB_REQUIRE(sp != nullptr, LUTB_ERR_NULL, "sparse index is NULL");
    LUTB_REQUIRE(sp->det_wbase && sp->det_stride && sp->det_count && sp->det_sstart && sp->syn_det && sp->syn_target &&
                     sp->chunk_info,
                 LUTB_ERR_NULL, "a sparse index array is NULL");
    LUTB_REQUIRE(sp->group_size > 0 && sp->n_syn_per_sample > 0 && sp->n_weights > 0 && sp->max_count > 0 &&
                     sp->n_chunks > 0,
                 LUTB_ERR_SHAPE, "empty sparse index");
    LUTB_REQUIRE((reinterpret_cast<uintptr_t>(sp->chunk_info) & 15) == 0, LUTB_ERR_ALIGN,
                 "chunk_info must be 16-byte aligned");
    return LUTB_OK;
}

static int chunk_grid(int64_t items, unsigned *blocks) {
    const int64_t n = (items + 7) / 8;  // 8 warps per block
    LUTB_REQUIRE(n <= 0x7FFFFFFF, LUTB_ERR_SHAPE, "batch too large for one launch");
    *blocks = (unsigned)n;
    return LUTB_OK;
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
    SparseView v = make_view(sp);
    unsigned blocks;
    rc = chunk_grid(batch * sp->n_chunks, &blocks);
    if (rc) return rc;
    {
        KernelScope scope(K_SPARSE_FORWARD, st);
        if (cfg->int_mode)
            sparse_forward_kernel<true><<<blocks, 256, 0, st>>>(v, weights, idx, y, batch, cfg->n_outputs, cfg->n_detectors, cfg->int_rescaler);
        else
            sparse_forward_kernel<false><<<blocks, 256, 0, st>>>(v, weights, idx, y, batch, cfg->n_outputs, cfg->n_detectors, cfg->int_rescaler);
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
        } else if (sp->max_count > 32) {
            unsigned blocks;
            rc = chunk_grid(batch * Nt, &blocks);
            if (rc) return rc;
            sparse_input_grad_long_kernel<<<blocks, 256, 0, st>>>(v, weights, dY, reinterpret_cast<const int2 *>(anchors), idx,
                                                                 min_delta, min_k, dX, batch, cfg->n_inputs, O, Nt, cfg->n_anchors);
        } else {
            unsigned blocks;
            rc = chunk_grid(batch * sp->n_chunks, &blocks);
            if (rc) return rc;
            const int2 *an = reinterpret_cast<const int2 *>(anchors);
            if (sp->max_count > 16)
                sparse_input_grad_kernel<32><<<blocks, 256, 0, st>>>(v, weights, dY, an, idx, min_delta, min_k, dX, batch, cfg->n_inputs, O, Nt, cfg->n_anchors);
            else if (sp->max_count > 8)
                sparse_input_grad_kernel<16><<<blocks, 256, 0, st>>>(v, weights, dY, an, idx, min_delta, min_k, dX, batch, cfg->n_inputs, O, Nt, cfg->n_anchors);
            else
                sparse_input_grad_kernel<8><<<blocks, 256, 0, st>>>(v, weights, dY, an, idx, min_delta, min_k, dX, batch, cfg->n_inputs, O, Nt, cfg->n_anchors);
        }
    }
    LUTB_LAUNCH_CHECK();
    double lr = cfg->lr_meta;
    if (external_lr >= 0.0) lr *= -(double)(float)external_lr;
    float *target = external_lr >= 0.0 ? weights : dW;
    {
        unsigned blocks;
        rc = chunk_grid(batch * sp->n_chunks, &blocks);
        if (rc) return rc;
        KernelScope scope(K_SPARSE_WEIGHT_GRAD, st);
        if (cfg->int_mode)
            sparse_weight_grad_kernel<true><<<blocks, 256, 0, st>>>(v, dY, idx, target, batch, O, Nt, lr, cfg->int_rescaler);
        else
            sparse_weight_grad_kernel<false><<<blocks, 256, 0, st>>>(v, dY, idx, target, batch, O, Nt, lr, cfg->int_rescaler);
    }
    LUTB_LAUNCH_CHECK();
    if (cfg->int_mode) {
        rc = launch_fixed_to_float(dX, batch * (int64_t)cfg->n_inputs, cfg->int_rescaler, st);
        if (rc) return rc;
        if (dW) rc = launch_fixed_to_float(dW, sp->n_weights, cfg->int_rescaler, st);
    }
    return rc;
}
